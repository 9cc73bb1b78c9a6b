// Device-side small-message exchange between the ranks of one box.  Every rank owns a mailbox arena that all
// peers have mapped; a message is written into every peer's arena with plain stores, fenced at system scope
// and announced with a release store of a monotonically increasing epoch tag.  Two parities alternate so a
// fast rank can never overwrite a message that a slow rank has not read yet (a rank can only be one exchange
// ahead, because finishing an exchange needs every peer's message of that exchange).  Replaces the
// host-mediated AllReduceThroughMaster / best-split read-back of the reference
// (catboost/cuda/cuda_lib/cuda_buffer_helpers/all_reduce.h:52-68, catboost/cuda/methods/histograms_helper.h:322-331).
// All waits are bounded (cb_wait_flag); a timeout sets the status word and the kernel carries on.
#pragma once
#include "cb_common.cuh"

// Small all-reduce / all-gather through the peer-mapped mailboxes (one block).
static __device__ void cb_mailbox_exchange(const CbComm& c, const void* src, int bytes, unsigned long long* epoch_out) {
    __shared__ unsigned long long s_epoch;
    if (threadIdx.x == 0) { s_epoch = c.epoch[0] + 1; c.epoch[0] = s_epoch; }
    __syncthreads();
    const unsigned long long epoch = s_epoch;
    const int parity = (int)(epoch & 1ull);
    const int words = (bytes + 7) >> 3;
    const unsigned long long* s = reinterpret_cast<const unsigned long long*>(src);
    for (int r = 0; r < c.nranks; ++r) {
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(
            c.peer_mbox[r] + (size_t)(parity * c.nranks + c.rank) * c.mbox_bytes);
        for (int i = threadIdx.x; i < words; i += blockDim.x) dst[i] = s[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < c.nranks) cb_st_release_sys(c.peer_mbox_flag[threadIdx.x] + parity * c.nranks + c.rank, epoch);
    if (threadIdx.x < c.nranks)
        cb_wait_flag(c.peer_mbox_flag[c.rank] + parity * c.nranks + threadIdx.x, epoch, c.timeout_ns, c.status,
                     CB_TIMEOUT_MAILBOX, (int)threadIdx.x);
    __syncthreads();
    *epoch_out = epoch;
}
__device__ __forceinline__ const char* cb_mailbox_msg(const CbComm& c, unsigned long long epoch, int src) {
    return c.peer_mbox[c.rank] + (size_t)((int)(epoch & 1ull) * c.nranks + src) * c.mbox_bytes;
}

// vals[count] (doubles in local global memory) <- sum over ranks, added in rank order on every rank.
static __device__ void cb_mailbox_allreduce_sum(const CbComm& c, double* vals, int count) {
    if (c.nranks <= 1) return;
    unsigned long long epoch;
    cb_mailbox_exchange(c, vals, count * 8, &epoch);
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        double s = 0.0;
        for (int r = 0; r < c.nranks; ++r) s += __ldcg(reinterpret_cast<const double*>(cb_mailbox_msg(c, epoch, r)) + i);
        vals[i] = s;
    }
    __syncthreads();
}


// ---- tagged words ("low latency" messages) ---------------------------------------------------------------
// A 32-bit payload travels together with a 32-bit tag in one 8-byte store, which is single-copy atomic also through
// a peer mapping: the reader polls the word itself until the tag is the one it expects, so a message needs neither
// a system-scope fence nor a separate flag (one NVLink hop instead of store + fence + flag + poll).  The tag is the
// low half of a monotonically increasing epoch, never 0; buffers start out zeroed.  A buffer may only be rewritten
// when every reader of its previous content is known to be done (the callers alternate two parities and rely on the
// fact that a rank cannot run more than one exchange ahead of a peer it needs an answer from).
__device__ __forceinline__ void cb_ll_store(unsigned long long* dst, unsigned int payload, unsigned int tag) {
    const unsigned long long v = ((unsigned long long)tag << 32) | (unsigned long long)payload;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long cb_ll_peek(const unsigned long long* src) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(src) : "memory");
    return v;
}
// Payload of the word once its tag is `tag`.  Bounded: after timeout_ns the status word is set and 0 is returned.
__device__ __forceinline__ unsigned int cb_ll_load(const unsigned long long* src, unsigned int tag, long long timeout_ns,
                                                   int* status, int code, int detail) {
    unsigned long long v = cb_ll_peek(src);
    if ((unsigned int)(v >> 32) == tag) return (unsigned int)v;
    const unsigned long long t0 = cb_globaltimer();
    unsigned int spins = 0;
    for (;;) {
        v = cb_ll_peek(src);
        if ((unsigned int)(v >> 32) == tag) return (unsigned int)v;
        if ((++spins & 63u) == 0u && (long long)(cb_globaltimer() - t0) > timeout_ns) {
            if (atomicCAS(status, CB_OK, code) == CB_OK) status[1] = detail;
            return 0u;
        }
    }
}
// Tag of an epoch: never 0, so a zero-filled buffer never looks delivered.
__device__ __forceinline__ unsigned int cb_ll_tag(unsigned long long epoch) {
    const unsigned int t = (unsigned int)epoch;
    return t ? t : 0x80000000u;
}
// Mailbox area of (parity, source rank) in rank `owner`'s arena, as tagged words.
__device__ __forceinline__ unsigned long long* cb_ll_box(const CbComm& c, int owner, int parity, int src) {
    return reinterpret_cast<unsigned long long*>(c.peer_mbox[owner] + (size_t)(parity * c.nranks + src) * c.mbox_bytes);
}
