"""Request-level data parallelism: one process per GPU, weights replicated, requests dealt round-robin, no collective
on the token loop. The only communication is one all_gather of a fixed-size stats vector at the end (NCCL on GPUs,
gloo in CPU tests) and the barriers that bracket a timed region.

The reference is single-GPU (no torch.distributed anywhere in it); this is the multi-GPU form the benchmark definition
asks for: request i goes to rank i mod world_size, each rank runs its own 128-slot StreamDecoder and scheduler.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

STAT_FIELDS = ("steps", "row_steps", "padded_row_steps", "slot_steps", "admitted", "evicted", "new_tokens",
               "delivered_tokens", "bytes", "h2d_bytes", "d2h_bytes", "elapsed_us", "gpu_us", "steady_row_steps",
               "steady_slot_steps", "p50_step_ns")


def env_world() -> tuple[int, int, int]:
    """(rank, local_rank, world_size) from the torchrun environment (1 process when absent)."""
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def init(backend: str | None = None) -> tuple[int, int, int]:
    rank, local, world = env_world()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep NCCL's banner off stdout (one JSON line there)
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return rank, local, world


def partition(requests: list, rank: int, world: int) -> list:
    """Round-robin: request i belongs to rank i mod world. Arrival times are rescaled so each rank keeps the stream's
    rate per GPU (a rank sees every world-th arrival, so its clock runs world times slower)."""
    mine = []
    for i in range(rank, len(requests), world):
        r = requests[i]
        c = type(r)(**vars(r))
        c.arrival = r.arrival / world
        mine.append(c)
    return mine


def gather_stats(stats: dict, device: torch.device | str = "cpu") -> list[dict]:
    """Every rank's stats (STAT_FIELDS, missing = 0) on every rank; one all_gather of 16 int64."""
    vec = torch.tensor([int(stats.get(k, 0)) for k in STAT_FIELDS], dtype=torch.int64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        out = [torch.zeros_like(vec) for _ in range(dist.get_world_size())]
        dist.all_gather(out, vec)
    else:
        out = [vec]
    return [dict(zip(STAT_FIELDS, (int(x) for x in v.cpu().tolist()))) for v in out]


def barrier(device=None) -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        if device is not None and torch.device(device).type == "cuda":
            dist.barrier(device_ids=[torch.device(device).index])
        else:
            dist.barrier()


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def check_identical(digest: str, device: torch.device | str = "cpu") -> None:
    """Every rank holds the same packed weights: one all_gather of the 32-byte SHA-256 digest
    (StreamDecoder.weights_digest); raises on the ranks that differ from rank 0."""
    mine = torch.tensor(list(bytes.fromhex(digest)), dtype=torch.uint8, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        out = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(out, mine)
        if not torch.equal(out[0], mine):
            raise RuntimeError(f"rank {dist.get_rank()}: packed weights differ from rank 0's "
                               f"({digest[:16]}... vs {bytes(out[0].cpu().tolist()).hex()[:16]}...)")
