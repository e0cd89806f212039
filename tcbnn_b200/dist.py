"""Multi-GPU plumbing of the batch-sharded forward pass: one process per GPU, every rank runs
the whole network on its own images, and the only exchange is one all-gather of the fp32 logits
(the reference's harness does one ncclReduce over the logits, benn_scaleup.cu:388-403).
Backend "nccl" on GPUs; "gloo" lets the same code run on CPU tensors in the tests."""
import os

import torch
import torch.distributed as dist


def init(backend=None, device=None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.
    Returns (rank, world).  A single process needs no group."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        kw = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return rank, world


def shard_seed(base_seed, rank):
    """Image seed of a rank's shard: shards differ, weights (seeded separately) do not."""
    return base_seed + rank


def shard_range(total_images, rank, world):
    """[begin, end) of the images rank owns when `total_images` are split evenly."""
    per = total_images // world
    if per * world != total_images:
        raise ValueError("batch %d does not split over %d ranks" % (total_images, world))
    return rank * per, (rank + 1) * per


def gather_logits(local, out=None):
    """All-gather [B][classes] logits into [world*B][classes], rank-major."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    if out is None:
        out = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                          device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous())
    return out


def ensemble_max(local, root=0):
    """The reference harness's own exchange (benn_scaleup.cu:400, benn_scaleout.cu): every rank
    holds a member network's [B][classes] logits for the SAME images and rank `root` ends with
    their element-wise maximum -- one reduce(max), in place.  Other ranks' tensors keep their
    own values.  Returns `local`."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.reduce(local, dst=root, op=dist.ReduceOp.MAX)
    return local


def max_over_ranks(values, device=None):
    """Element-wise max of a list of floats over all ranks (timings are reported as the max)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def barrier():
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def finish():
    if dist.is_initialized():
        dist.destroy_process_group()
