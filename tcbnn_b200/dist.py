"""Multi-GPU plumbing of the batch-sharded forward pass: one process per GPU, every rank runs
the whole network on its own images, and the only exchange is one all-gather of the fp32 logits
(the reference's harness does one ncclReduce over the logits, benn_scaleup.cu:388-403).
Backend "nccl" on GPUs; "gloo" lets the same code run on CPU tensors in the tests."""
import os

import torch
import torch.distributed as dist


def init(backend=None, device=None, timeout_s=None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.
    Returns (rank, world).  A single process needs no group.  timeout_s: how long a collective may
    take before it raises (the backend's default otherwise)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        kw = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        if timeout_s:
            import datetime
            kw["timeout"] = datetime.timedelta(seconds=float(timeout_s))
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


class OverlappedGather:
    """gather_logits() off the compute stream: step i's logits are copied into one of two staging
    buffers on the compute stream (4 MB, device to device) and gathered from there on a side
    stream while step i+1 computes; the compute stream only waits before it reuses a staging
    buffer, i.e. for the gather of two steps ago.  On CPU tensors (gloo, tests) the gather is
    done in place, synchronously.  finish() makes the compute stream wait for what is in flight."""

    def __init__(self, rows, cols, dtype, device, world):
        self.world = world
        self.cuda = torch.device(device).type == "cuda"
        self.out = torch.empty((world * rows, cols), dtype=dtype, device=device)
        if self.cuda and world > 1:
            self.stage = [torch.empty((rows, cols), dtype=dtype, device=device) for _ in range(2)]
            self.side = torch.cuda.Stream(device=device)
            self.staged = [torch.cuda.Event() for _ in range(2)]
            self.gathered = [torch.cuda.Event() for _ in range(2)]
            self.used = [False, False]
        self.n = 0

    def __call__(self, local):
        if self.world == 1:
            return local
        if not self.cuda:
            return gather_logits(local, self.out)
        k = self.n & 1
        self.n += 1
        main = torch.cuda.current_stream()
        if self.used[k]:
            main.wait_event(self.gathered[k])            # the gather that last read this buffer
        self.stage[k].copy_(local, non_blocking=True)
        self.staged[k].record(main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(self.staged[k])
            dist.all_gather_into_tensor(self.out, self.stage[k])
            self.gathered[k].record(self.side)
        self.used[k] = True
        return self.out

    def finish(self):
        if self.world > 1 and self.cuda:
            for k in range(2):
                if self.used[k]:
                    torch.cuda.current_stream().wait_event(self.gathered[k])
        return self.out


def pin_to_gpu_node(local_rank, local_world):
    """Restrict this process to a share of the CPU cores of its GPU's NUMA node, so that the
    pinned host buffers it allocates afterwards are first touched there and the ranks of one box
    do not crowd onto the same cores (the launcher leaves every rank on all of them).  Returns the
    list of cores, or None when the topology cannot be read (nothing is changed then)."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = -1
        path = "/sys/bus/pci/devices/%s/numa_node" % bdf
        if os.path.exists(path):
            node = int(open(path).read().strip())
        allowed = sorted(os.sched_getaffinity(0))
        cpus = allowed
        if node >= 0:
            txt = open("/sys/devices/system/node/node%d/cpulist" % node).read().strip()
            on_node = set()
            for part in txt.split(","):
                lo, _, hi = part.partition("-")
                on_node.update(range(int(lo), int(hi or lo) + 1))
            cpus = [c for c in allowed if c in on_node] or allowed
        share = max(1, len(cpus) // max(1, local_world))
        mine = cpus[local_rank * share:(local_rank + 1) * share] or cpus
        os.sched_setaffinity(0, mine)
        return mine
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


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
