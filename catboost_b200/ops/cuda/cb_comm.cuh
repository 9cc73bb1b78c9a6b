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

