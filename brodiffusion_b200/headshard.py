"""Head-sharded attention across the GPUs of one node.

Heads are independent, so GPU g of G owns the contiguous head range
``head_range(num_heads, G, g)`` and needs no data from its peers until the
output projection, which consumes all heads.  The one exchange step is an
all-gather of the per-head outputs over NVLink (NCCL).  Each rank writes its
attention output into its own slab of a head-major staging tensor
``(G, B, L, heads_per_gpu * head_dim)`` and the all-gather runs in place on
that tensor, so no re-layout copy is made; the output projection reads the
staging tensor slab by slab (``project_staged``), which is the same matrix
product as ``(B, L, D) @ Wo^T`` with its K dimension walked in G blocks.

The reference has no multi-GPU path (it is single-device); this module is the
B200 addition for the long-sequence Flux configuration.
"""
from __future__ import annotations


def head_range(num_heads: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, equal head ranges; ``world`` must divide ``num_heads``."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"head_range: bad rank {rank} of {world}")
    if num_heads % world != 0:
        raise ValueError(f"head_range: {world} GPUs do not divide {num_heads} heads")
    per = num_heads // world
    return rank * per, (rank + 1) * per


def staging_shape(world: int, batch: int, rows: int, num_heads: int, head_dim: int):
    return (world, batch, rows, (num_heads // world) * head_dim)


def all_gather_heads(staging, group=None):
    """In-place all-gather of the staging tensor: slab ``rank`` holds this
    rank's output on entry; every slab is filled on return."""
    import torch.distributed as dist
    rank = dist.get_rank(group)
    G, B = staging.shape[0], staging.shape[1]
    flat = staging.view(G * B, *staging.shape[2:])      # slabs concatenated along dim 0
    dist.all_gather_into_tensor(flat, staging[rank], group=group)
    return staging


def unstage(staging):
    """(G, B, L, d) -> (B, L, G*d): the row-major layout of the reference's
    attention output (used by tests; the product path projects from the
    staging layout directly)."""
    G, B, L, d = staging.shape
    return staging.permute(1, 2, 0, 3).reshape(B, L, G * d)


def project_staged(staging, w_out, bias=None):
    """Output projection from the staging layout: sum over slabs g of
    ``staging[g] @ w_out[:, g*d:(g+1)*d]^T``."""
    import torch
    G, B, L, d = staging.shape
    y = None
    for g in range(G):
        part = torch.matmul(staging[g], w_out[:, g * d:(g + 1) * d].t())
        y = part if y is None else y + part
    if bias is not None:
        y = y + bias
    return y


class GatheredOutput:
    """Full (B, L, D) attention output replicated on every rank in symmetric
    memory, for the fused all-gather (``bdattn_sdpa_fwd_allgather``): each rank's
    attention kernel stores its head columns into every replica (through
    peer-mapped pointers, or once through the switch's multicast address), so after ``barrier()`` every rank holds the reference
    layout (B, L, num_heads * head_dim) without a staging copy or an NCCL call.
    """

    def __init__(self, batch, rows, num_heads, head_dim, dtype, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.h0, self.h1 = head_range(num_heads, self.world, self.rank)
        self.head_dim = head_dim
        self.full = symm_mem.empty((batch, rows, num_heads * head_dim), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.full, self.group)
        self.col0 = self.h0 * head_dim
        self.elem = self.full.element_size()
        # this rank's head columns inside its own replica
        self.local = self.full[:, :, self.col0:self.h1 * head_dim]
        self.peer_bases = [int(self.handle.buffer_ptrs[r]) for r in range(self.world) if r != self.rank]
        # NVLink multicast address of the replicas (0 when the group has no switch multicast)
        self.multicast_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def peer_ptrs(self, row0=0):
        """Peer addresses of element (0, row0, first own column)."""
        D = self.full.shape[2]
        off = (row0 * D + self.col0) * self.elem
        return [b + off for b in self.peer_bases]

    def multicast_ptr(self, row0=0):
        """Multicast address of element (0, row0, first own column): a store to it
        lands in every rank's replica.  None without switch multicast."""
        if not self.multicast_base:
            return None
        D = self.full.shape[2]
        return self.multicast_base + (row0 * D + self.col0) * self.elem

    def barrier(self):
        """Stream-ordered cross-GPU barrier: once it has passed on this rank's
        stream, every rank's attention kernel enqueued before its own barrier
        has completed, so all head columns of the local replica are written."""
        self.handle.barrier()
