"""Multi-GPU entry: one process per GPU.

``fit(task_type='GPU', devices='0-7')`` from a plain Python process spawns one worker per device; each worker joins a
``torch.distributed`` NCCL group on 127.0.0.1, takes a contiguous row shard (query groups are kept whole, like
catboost/cuda/gpu_data/doc_parallel_dataset_builder.cpp:20-55), trains doc-parallel and rank 0 hands the result back.
The data set reaches the workers through POSIX shared memory: the parent copies every large array of the pool once
into a shared segment, a worker maps the segments and looks at its own rows only (views, no copy), so host memory
holds two copies of the data in total whatever the number of GPUs (the reference keeps one copy because its workers are
threads of one process).
When the caller already runs under ``torchrun`` (torch.distributed initialised, world size > 1) ``fit`` is a
collective call: every rank passes its own row shard and all ranks return the same model.
"""
from __future__ import annotations

import os
import pickle
import socket
import tempfile
from typing import List, Optional

import numpy as np
import torch

from ..data.pool import CatBoostError, Pool
from ..params import normalize_params, parse_devices
from .runtime import DistContext


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def shard_bounds(pool: Pool, world: int) -> List[int]:
    """Row boundaries of ``world`` contiguous shards; a query group never straddles a boundary."""
    n = pool.num_row()
    if pool.group_id is None:
        return [n * r // world for r in range(world + 1)]
    off = pool.group_offsets()
    bounds = [0]
    for r in range(1, world):
        target = n * r / world
        k = int(np.searchsorted(off, target))
        k = min(max(k, 0), len(off) - 1)
        bounds.append(int(max(off[k], bounds[-1])))
    bounds.append(n)
    return bounds


_SHARED_ATTRS = ("float_data", "cat_hashes", "label", "weight", "group_weight", "baseline", "timestamp", "group_id",
                 "subgroup_id", "pairs", "pairs_weight")


def share_pool(pool: Pool):
    """(descriptor, segments): the large numeric arrays of ``pool`` copied into shared-memory segments, everything else
    (names, indices, text columns) pickled inside the descriptor.  The caller unlinks the segments when done."""
    from multiprocessing import shared_memory
    segments, arrays = [], {}
    small = dict(pool.__dict__)
    small.pop("_cat_hash_tensors", None)
    small["_quantized"] = None
    small["_cat_distinct"] = {}

    def put(key, arr):
        a = np.ascontiguousarray(arr)
        seg = shared_memory.SharedMemory(create=True, size=max(1, a.nbytes))
        np.ndarray(a.shape, dtype=a.dtype, buffer=seg.buf)[...] = a
        segments.append(seg)
        arrays[key] = (seg.name, a.shape, a.dtype.str)

    for k in _SHARED_ATTRS:
        v = small.get(k)
        if isinstance(v, np.ndarray) and v.dtype.kind in "fiub" and v.nbytes >= (1 << 16):
            put(k, v)
            small[k] = None
    emb = list(small.get("embedding_data") or [])
    for j, e in enumerate(emb):
        if isinstance(e, np.ndarray) and e.dtype.kind in "fiub":
            put(f"embedding_data:{j}", e)
            emb[j] = None
    small["embedding_data"] = emb
    return {"small": pickle.dumps(small, protocol=4), "arrays": arrays}, segments


def attach_pool(desc):
    """Pool whose large arrays are views of the shared segments named in ``desc`` (+ the handles to keep alive)."""
    from multiprocessing import shared_memory
    pool = Pool.__new__(Pool)
    pool.__dict__.update(pickle.loads(desc["small"]))
    handles = []
    for key, (name, shape, dt) in desc["arrays"].items():
        seg = shared_memory.SharedMemory(name=name)
        try:
            # the segment belongs to the parent: keep this process's exit from unlinking it
            from multiprocessing import resource_tracker
            resource_tracker.unregister(seg._name, "shared_memory")
        except Exception:
            pass
        handles.append(seg)
        arr = np.ndarray(shape, dtype=np.dtype(dt), buffer=seg.buf)
        if key.startswith("embedding_data:"):
            pool.embedding_data[int(key.split(":")[1])] = arr
        else:
            setattr(pool, key, arr)
    return pool, handles


def _worker(rank: int, world: int, port: int, devices, params, pool_blob_path, eval_blob_paths, default_loss, out_path,
            backend: str):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["LOCAL_RANK"] = str(rank)
    if backend == "nccl":
        torch.cuda.set_device(devices[rank])
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", devices[rank]))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ..train.boosting import train_model
        keep = []
        with open(pool_blob_path, "rb") as fh:
            pool, hs = attach_pool(pickle.load(fh))
        keep += hs
        b = shard_bounds(pool, world)
        shard = pool.slice_range(b[rank], b[rank + 1])
        evals = []
        for p in eval_blob_paths:
            with open(p, "rb") as fh:
                ep, hs = attach_pool(pickle.load(fh))
            keep += hs
            eb = shard_bounds(ep, world)
            evals.append(ep.slice_range(eb[rank], eb[rank + 1]))
        params = dict(params)
        params["devices"] = ":".join(str(d) for d in devices)
        res = train_model(params, shard, evals, default_loss=default_loss, ctx=DistContext.current())
        if rank == 0:
            res.options = dict(res.options)
            res.options.pop("callback", None)
            with open(out_path, "wb") as fh:
                pickle.dump(res, fh, protocol=4)
    finally:
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()
        try:
            del shard, evals, pool
        except NameError:
            pass
        for seg in locals().get("keep", []):
            try:
                seg.close()
            except BufferError:
                pass


def train_maybe_multi_gpu(params, train_pool: Pool, eval_pools, default_loss="RMSE", init_model=None, callbacks=None,
                          log_cout=None):
    from ..train.boosting import train_model
    ctx = DistContext.current()
    p = normalize_params(params)
    task = str(p.get("task_type", "CPU")).upper()
    if ctx.is_distributed or task != "GPU":
        return train_model(params, train_pool, eval_pools, default_loss=default_loss, init_model=init_model, ctx=ctx,
                           callbacks=callbacks, log_cout=log_cout)
    if not torch.cuda.is_available():
        raise CatBoostError("task_type='GPU' was requested but no CUDA device is available")
    devices = parse_devices(p.get("devices"), torch.cuda.device_count()) if p.get("devices") is not None else [0]
    if len(devices) <= 1:
        return train_model(params, train_pool, eval_pools, default_loss=default_loss, init_model=init_model, ctx=ctx,
                           callbacks=callbacks, log_cout=log_cout)
    if init_model is not None or callbacks:
        raise CatBoostError("init_model and callbacks are not supported with several devices from one process; "
                            "launch with torchrun instead")
    return spawn_training(params, train_pool, eval_pools, devices, default_loss, backend="nccl")


def spawn_training(params, train_pool, eval_pools, devices, default_loss="RMSE", backend="nccl"):
    """Run doc-parallel training in ``len(devices)`` child processes and return rank 0's result."""
    import torch.multiprocessing as mp
    world = len(devices)
    tmp = tempfile.mkdtemp(prefix="cb200_")
    pool_path = os.path.join(tmp, "train.pkl")
    segments = []
    desc, segs = share_pool(train_pool)
    segments += segs
    with open(pool_path, "wb") as fh:
        pickle.dump(desc, fh, protocol=4)
    eval_paths = []
    for k, ep in enumerate(eval_pools):
        pth = os.path.join(tmp, f"eval{k}.pkl")
        desc, segs = share_pool(ep)
        segments += segs
        with open(pth, "wb") as fh:
            pickle.dump(desc, fh, protocol=4)
        eval_paths.append(pth)
    out_path = os.path.join(tmp, "result.pkl")
    port = _free_port()
    params = {k: v for k, v in dict(params).items() if k != "callback"}
    try:
        mp.spawn(_worker, args=(world, port, list(devices), params, pool_path, eval_paths, default_loss, out_path,
                                backend), nprocs=world, join=True)
        with open(out_path, "rb") as fh:
            res = pickle.load(fh)
        from ..params import Options
        res.options = Options(res.options)
        return res
    finally:
        for seg in segments:
            try:
                seg.close()
                seg.unlink()
            except (OSError, BufferError):
                pass
        for f in [pool_path, out_path] + eval_paths:
            try:
                os.remove(f)
            except OSError:
                pass
        try:
            os.rmdir(tmp)
        except OSError:
            pass
