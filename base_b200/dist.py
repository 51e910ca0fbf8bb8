"""Multi-process plumbing, one process per GPU: the barrier / max / sum the
benchmark contract asks for, the hand-out of the communicator id for the
expert-parallel decode step, and a host restatement of that step's exchange
(`ep_moe_layer`) which the CPU tests run on gloo ranks and the GPU tests compare
the device path with.  Backend `nccl` on GPUs, `gloo` in the CPU tests.

The reference has no multi-device path.  Experts are independent given the
routed tokens (lean/lib/AlgorithmLib/ML/Compose.lean:1812-1828): rank r owns
experts [r E / W, (r + 1) E / W) (`expert_range`) and `batch` of the sequences.
Per MoE layer: (1) every rank sends its tokens' normalised hidden states to
every rank (the dispatch all-to-all at full capacity = an all-gather); (2) every
rank routes all tokens (replicated router) and runs its experts on the tokens
routed to them; (3) per token it adds its experts' outputs, weighted, in top-k
order; (4) an all-to-all returns each sequence's partial sums to its owner, who
adds them in rank order.  The device path does the same inside one CUDA graph
(csrc/stages/gptoss_batch.inc) with NCCL from the C ABI.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple


class Ranks:
    """Thin wrapper over torch.distributed that degrades to one process."""

    def __init__(self, backend: Optional[str] = None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self._dist = None
        self._device = "cpu"
        if self.world > 1:
            import torch
            import torch.distributed as dist
            backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            if backend == "nccl":
                torch.cuda.set_device(self.local)
                self._device = f"cuda:{self.local}"
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            else:
                dist.init_process_group(backend)
            self._dist = dist

    def barrier(self) -> None:
        if self._dist is not None:
            self._dist.barrier()

    def _reduce(self, v: float, op: str) -> float:
        if self._dist is None:
            return float(v)
        import torch
        t = torch.tensor([v], device=self._device, dtype=torch.float64)
        self._dist.all_reduce(t, op=getattr(self._dist.ReduceOp, op))
        return float(t.item())

    def max(self, v: float) -> float:
        return self._reduce(v, "MAX")

    def sum(self, v: float) -> float:
        return self._reduce(v, "SUM")

    def all_reduce_sum(self, tensor) -> None:
        """In-place sum of a torch tensor over the ranks (the expert-parallel combine)."""
        if self._dist is not None:
            self._dist.all_reduce(tensor, op=self._dist.ReduceOp.SUM)

    def throughput(self, units_local: float, seconds_local: float) -> float:
        """Whole-job rate: every rank's units over the slowest rank's time."""
        return self.sum(units_local) / self.max(seconds_local)

    def broadcast_bytes(self, payload: Optional[bytes]) -> bytes:
        """Rank 0's bytes on every rank (the communicator id for GptOss.comm_init)."""
        if self._dist is None:
            return payload or b""
        box = [payload if self.rank == 0 else None]
        self._dist.broadcast_object_list(box, src=0)
        return box[0]

    def all_gather_bytes(self, payload: bytes) -> list:
        """Every rank's bytes on every rank, in rank order (the memory handles for GptOss.peer_init)."""
        if self._dist is None:
            return [payload]
        box = [None] * self.world
        self._dist.all_gather_object(box, payload)
        return box

    def all_gather_rows(self, rows):
        """numpy [n, H] per rank -> [world * n, H], rank order (host path of the dispatch)."""
        if self._dist is None:
            return rows
        import numpy as np
        import torch
        t = torch.from_numpy(np.ascontiguousarray(rows)).to(self._device)
        out = [torch.empty_like(t) for _ in range(self.world)]
        self._dist.all_gather(out, t)
        return np.concatenate([o.cpu().numpy() for o in out], axis=0)

    def all_to_all_rows(self, rows):
        """numpy [world, n, H]: chunk q goes to rank q; returns [world, n, H] with chunk q from rank q."""
        if self._dist is None:
            return rows
        import numpy as np
        import torch
        send = [torch.from_numpy(np.ascontiguousarray(rows[q])).to(self._device) for q in range(self.world)]
        recv = [torch.empty_like(send[0]) for _ in range(self.world)]
        if self._device == "cpu":
            # gloo has no all-to-all for CPU tensors: pairwise exchange, lower rank sends first
            for q in range(self.world):
                if q == self.rank:
                    recv[q].copy_(send[q])
                elif self.rank < q:
                    self._dist.send(send[q], q)
                    self._dist.recv(recv[q], q)
                else:
                    self._dist.recv(recv[q], q)
                    self._dist.send(send[q], q)
        else:
            self._dist.all_to_all(recv, send)
        return np.stack([r.cpu().numpy() for r in recv])

    def close(self) -> None:
        if self._dist is not None:
            self._dist.destroy_process_group()
            self._dist = None


def expert_range(rank: int, world: int, experts: int) -> Tuple[int, int]:
    """Experts [lo, lo + n) owned by `rank` under expert-parallel sharding
    (contiguous blocks; `world` must divide `experts`)."""
    if world <= 0 or experts % world:
        raise ValueError("world size must divide the number of experts")
    n = experts // world
    return rank * n, n


def ep_moe_layer(ranks: "Ranks", xn_local, experts: int, top_k: int, route_fn, expert_fn):
    """Host restatement of one expert-parallel MoE layer for this rank's tokens.

    xn_local [n, H] f32: this rank's normalised hidden states.  route_fn(x_all) -> (idx [T, k], w [T, k]) is the
    replicated router; expert_fn(e, x_row) -> [H] runs expert e (called only for this rank's experts).  Returns
    y [n, H]: for every local token the sum over ranks (ascending) of that rank's partial sum, each partial sum
    being the rank's experts' outputs times their gates, added in top-k order.
    """
    import numpy as np
    lo, n_e = expert_range(ranks.rank, ranks.world, experts)
    x_all = ranks.all_gather_rows(np.asarray(xn_local, dtype=np.float32))
    idx, w = route_fn(x_all)
    T, H = x_all.shape
    part = np.zeros((T, H), dtype=np.float32)
    for t in range(T):
        for j in range(top_k):
            e = int(idx[t, j])
            if lo <= e < lo + n_e:
                part[t] = (part[t] + np.float32(w[t, j]) * expert_fn(e, x_all[t])).astype(np.float32)
    n = T // ranks.world
    got = ranks.all_to_all_rows(part.reshape(ranks.world, n, H))
    y = np.zeros((n, H), dtype=np.float32)
    for q in range(ranks.world):
        y = (y + got[q]).astype(np.float32)
    return y
