"""Axial (row / column) sharding of the pair tensor over the GPUs of one node, for complexes whose ``[N, N, C]`` pair
activations are too large or too slow for one GPU.

The reference has no such mode (it scales ``N`` on one GPU by row chunking, model/primitives.py:309-388); its
unsharded Pairformer block (model/evoformer.py:270-355) is the oracle. Layout and data movement:

* The resident layout is a **row shard**: rank ``p`` of ``P`` holds rows ``[p n, (p + 1) n)`` of ``z``, ``n = N / P``,
  as ``[B, n, N, C]``. Residual stream, transitions and every element-wise step work on it locally.
* The triangle multiplies contract over a token index but never over channels: ``out[c, i, j] = sum_k a[c, i, k]
  b[c, j, k]`` (outgoing) or ``sum_k a[c, k, j] b[c, k, i]`` (incoming). The gated ``a`` / ``b`` projections are
  written channel-major, an all-to-all turns "all channels of my rows" into "all rows of my ``C / P`` channels", every
  rank contracts its channels as full ``N x N x N`` products, and a second all-to-all brings the result back to rows
  for the channel LayerNorm. Each rank sends ``3 N^2 C / P`` elements per multiply, whatever the direction; gathering
  ``b`` instead would move ``N^2 C`` per rank.
* Triangle attention along rows ("starting node") is local per row; only its bias ``[H, N, N]``, a function of all of
  ``z``, is gathered (``H N^2 / P`` elements per rank, 32 times smaller than ``z``). Attention along columns ("ending
  node") runs on the column shard and its update is transposed back.
* The single track is replicated; its pair bias is gathered like the attention bias.

So one block moves six plane all-to-alls, two shard transposes and three bias gathers. ``AxialComm`` does them either
with ``torch.distributed`` collectives (any backend; the correctness oracle, and the path CPU tests run over gloo) or
with this package's peer-memory exchange kernel (``ops/csrc/peer_exchange.cu``: producer-side peer stores plus
bounded flag waits, no NCCL call).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import ops
from .dist import DistInfo, on_one_node


class AxialComm:
    """The four re-layouts of the sharded block. ``transport="peer"`` runs them on this package's peer-memory kernels
    (CUDA tensors, one node); ``"collective"`` states them with ``torch.distributed`` collectives on any backend."""

    def __init__(self, info: DistInfo, transport: str | None = None):
        self.info = info
        default = "collective"
        if info.is_distributed and info.backend == "nccl" and transport is None and "DF3_AXIAL_COMM" not in os.environ:
            default = "peer" if on_one_node(info) else "collective"  # peer mappings exist only inside one host
        self.transport = transport or os.environ.get("DF3_AXIAL_COMM", default)
        if self.transport not in ("peer", "collective"):
            raise ValueError(f"axial transport must be peer|collective, got {self.transport!r}")
        self._heap = None

    @property
    def world(self) -> int:
        return self.info.world_size

    @property
    def rank(self) -> int:
        return self.info.rank

    def rows(self, n_total: int) -> slice:
        n = n_total // self.world
        return slice(self.rank * n, (self.rank + 1) * n)

    def peer(self):
        if self._heap is None:
            from .peer_exchange import PeerExchange

            self._heap = PeerExchange(self.info)
        return self._heap

    def _on_peer(self, x) -> bool:
        return self.transport == "peer" and x.is_cuda

    def _all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        """``send[q]`` goes to rank ``q``; slot ``p`` of the result came from rank ``p``."""
        recv = torch.empty_like(send)
        if self.info.backend == "nccl":
            dist.all_to_all_single(recv, send)
        else:  # gloo has no all_to_all: one broadcast-free exchange through all_gather
            parts = [torch.empty_like(send) for _ in range(self.world)]
            dist.all_gather(parts, send)
            for p in range(self.world):
                recv[p] = parts[p][self.rank]
        return recv

    def check(self) -> None:
        if self._heap is not None:
            self._heap.check()

    # ------------------------------------------------------------------ re-layouts
    def all_gather(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        """Concatenate every rank's ``x`` along ``dim`` (rank order)."""
        if self.world == 1:
            return x
        if self._on_peer(x):
            return self.peer().all_gather(x, dim)
        xc = x.movedim(dim, 0).contiguous()
        parts = [torch.empty_like(xc) for _ in range(self.world)]
        dist.all_gather(parts, xc)
        return torch.cat(parts, 0).movedim(0, dim).contiguous()

    def transpose(self, x: torch.Tensor) -> torch.Tensor:
        """Row shard ``[B, n, N, C]`` of ``z`` -> row shard of ``z^T``: ``out[b, j_local, i] = z[b, i, rank * n + j_local]``.
        Applying it twice gives the input back."""
        P = self.world
        if P == 1:
            return x.transpose(1, 2).contiguous()
        if self._on_peer(x):
            return self.peer().transpose(x)
        B, n, N, C = x.shape
        # block q of the send buffer goes to rank q: z[i_local, q n + j_local] laid out [j_local, i_local]
        recv = self._all_to_all(x.view(B, n, P, n, C).permute(2, 0, 3, 1, 4).contiguous())  # [P, B, j_local, i_local, C]
        # block p came from rank p: its i_local are global rows p n + i_local
        return recv.permute(1, 2, 0, 3, 4).reshape(B, n, N, C)

    def rows_to_channels(self, x: torch.Tensor) -> torch.Tensor:
        """Channel planes of this rank's rows ``[G, C, B, n, N]`` -> all rows of channels ``[rank C/P, (rank + 1) C/P)`` of
        each of the ``G`` groups: ``[G, C / P, B, N, N]``."""
        P = self.world
        if P == 1:
            return x
        if self._on_peer(x):
            return self.peer().rows_to_channels(x)
        G, C, B, n, N = x.shape
        recv = self._all_to_all(x.view(G, P, C // P, B, n, N).movedim(1, 0).contiguous())  # [P (source), G, C/P, B, n, N]
        return recv.permute(1, 2, 3, 0, 4, 5).reshape(G, C // P, B, N, N)

    def channels_to_rows(self, x: torch.Tensor) -> torch.Tensor:
        """The way back: all rows of this rank's channels ``[C / P, B, N, N]`` -> all channels of this rank's rows
        ``[C, B, n, N]``."""
        P = self.world
        if P == 1:
            return x
        if self._on_peer(x):
            return self.peer().channels_to_rows(x)
        cp, B, N, _ = x.shape
        n = N // P
        recv = self._all_to_all(x.view(cp, B, P, n, N).permute(2, 0, 1, 3, 4).contiguous())  # [P (source), C/P, B, n, N]
        return recv.reshape(P * cp, B, n, N)


# ---------------------------------------------------------------------------------------------------------------------------
# Sharded forward of one Pairformer block (inference: no dropout, no autograd through the exchanges).
def _tri_mul_rows(mod, z_rows, mask_rows, comm: AxialComm):
    """Triangle multiply (either direction) on the row shard ``z_rows`` ``[B, n, N, C]``. Projections, gates and norms
    are local; the contraction runs on this rank's channels over all rows."""
    B, n, N, C = z_rows.shape
    if C % comm.world:
        raise ValueError(f"the pair width ({C}) must be a multiple of the number of ranks ({comm.world})")
    z0 = mod.norm_left(z_rows)
    nc = mod.norm_center
    nat = ops.fused(z0, "gated_dual_linear")
    native_planes = nat is not None and nat.has("plane_layer_norm") and nat.gemm_supported(z0, mod.gate.weight) and C in (32, 64, 128, 256)
    if native_planes:
        planes = nat.gated_dual_linear(z0, mod.gate.weight, mod.proj.weight, mask_rows, True, True).view(2, C, B, n, N)
    else:
        ab = ops.gated_dual_linear(z0, mod.gate.weight, mod.proj.weight, mask_rows)
        planes = torch.stack([ab[..., 0::2], ab[..., 1::2]]).permute(0, 4, 1, 2, 3).contiguous()  # [2, C, B, n, N]
    mine = comm.rows_to_channels(planes).flatten(1, 2)  # [2, (C / P) B, N, N]
    if native_planes:
        act = ops._plane_contract(nat, mine, mod.outgoing)
    else:
        a, b = mine[0], mine[1]
        act = torch.bmm(a, b.transpose(1, 2)) if mod.outgoing else torch.bmm(b.transpose(1, 2), a)
    act = comm.channels_to_rows(act.view(C // comm.world, B, N, N))  # [C, B, n, N]
    if mod.is_mhr:
        act = mod._head_mix(act.permute(1, 2, 3, 0), mod.router(z0) if mod.use_router else None)
    else:
        if native_planes:
            act = nat.plane_layer_norm(act.view(C, B * n * N), nc.weight, nc.bias, nc.eps).view(B, n, N, C)
        else:
            act = ops.layer_norm(act.permute(1, 2, 3, 0), nc.weight, nc.bias, nc.eps)
        if nc.output_scale != 1.0:
            act = act * nc.output_scale
    return ops.sigmoid_gate_mul(z0, mod.out_gate.weight, mod.out_proj(act))


def _attention_rows(mod, z_rows, key_mask_rows, bias_full):
    """Gated attention along the last token axis of ``z_rows`` ``[B, n, N, C]`` with the gathered bias ``[B, H, N, N]``."""
    B, n, N, _ = z_rows.shape
    H, D = mod.num_heads, mod.head_dim
    zn = mod.norm(z_rows)
    qkv = ops.stacked_linear(zn, mod.to_q.weight, mod.to_k.weight, mod.to_v.weight).view(B, n, N, 3, H, D)
    q, k, v = (qkv[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))  # [B, R = n, H, N, D]
    out = ops.pair_bias_attention(q, k, v, bias_full, key_mask_rows, mod.scale)
    out = out.permute(0, 1, 3, 2, 4).reshape(B, n, N, H * D)
    return mod.out_proj(ops.sigmoid_gate_mul(zn, mod.to_g.weight, out))


def _pair_updates(block, z, mask_rows, mask_cols, comm: AxialComm, gain, scale, transition_gain=1.0):
    """The pair half of a trunk block (both triangle multiplies, both triangle attentions, the transition) on rows."""
    z = z + gain * scale(_tri_mul_rows(block.tri_mul_out, z, mask_rows, comm))
    z = z + gain * scale(_tri_mul_rows(block.tri_mul_in, z, mask_rows, comm))
    if block.use_triangle_attention:
        row, col = block.pair_attn_row, block.pair_attn_col
        bias = comm.all_gather(ops.head_bias_planes(row.norm(z), row.pair_bias.weight), 2)  # [B, H, N, N]
        z = z + gain * scale(_attention_rows(row, z, mask_rows, bias))
        bias = comm.all_gather(ops.head_bias_planes(col.norm(z), col.pair_bias.weight), 2)
        zt = comm.transpose(z)
        z = z + comm.transpose(gain * scale(_attention_rows(col, zt, mask_cols, bias)))
    return z + gain * transition_gain * scale(block.pair_transition(z))


def _masks(pair_mask, comm: AxialComm):
    rows = comm.rows(pair_mask.shape[-1])
    # mask[i_local, j] for the row shard, mask[k, i_local] as the column shard sees it
    return pair_mask[:, rows], pair_mask.transpose(1, 2)[:, rows].contiguous()


@torch.no_grad()
def sharded_pairformer_block(block, pair_rows, single, pair_mask, seq_mask, comm: AxialComm):
    """One Pairformer block on a row shard. ``pair_rows`` ``[B, n, N, C]`` are this rank's rows of the pair tensor,
    ``pair_mask`` ``[B, N, N]`` and the single track are replicated. Returns ``(pair_rows, single)``; gathering the
    rows of all ranks gives what ``block(pair, single, pair_mask, seq_mask)`` gives in eval mode."""
    mask_rows, mask_cols = _masks(pair_mask, comm)
    s, scale = block.residual_out_scale, block.branch_scaler
    z = _pair_updates(block, pair_rows, mask_rows, mask_cols, comm, s, scale, block.pair_transition_residual_gain)
    if block.use_single_track:
        logits = ops.head_bias_planes(block.single_to_pair_norm(z), block.single_to_pair.weight)  # [B, Hs, n, N]
        logits = comm.all_gather(logits, 2)
        single = single + s * scale(block.single_attn(single, seq_mask, logits))
        single = single + s * block.single_transition_residual_gain * scale(block.single_transition(single))
    return z, single


@torch.no_grad()
def sharded_evoformer_block(block, msa, pair_rows, msa_mask, pair_mask, comm: AxialComm):
    """One MSA-stack block (reference: model/evoformer.py:84-177) with the pair tensor on row shards and the MSA
    replicated: the outer-product mean is computed for this rank's rows only, the MSA attention weights come from the
    local rows and are gathered (``[H, N, N]``), the MSA update itself is small and runs on every rank."""
    from ..models.primitives import map_row_chunks

    mask_rows, mask_cols = _masks(pair_mask, comm)
    rows = comm.rows(pair_mask.shape[-1])
    s = block.residual_out_scale
    opm = block.outer_product
    m = msa_mask.unsqueeze(-1)
    x = opm.norm(msa)
    a, b = opm.proj_a(x) * m.to(x.dtype), opm.proj_b(x) * m.to(x.dtype)
    z = pair_rows + s * ops.outer_product_mean(a[:, :, rows], b, opm.out_w, opm.out_b, None, mask_i=msa_mask[:, :, rows],
                                               mask_j=msa_mask)  # fmt: skip
    ra = block.row_attn
    logits = ra.pair_logits(ra.pair_norm(z)).permute(0, 3, 1, 2)  # [B, H, n, N]
    col_mask = msa_mask.max(dim=-2).values
    weights = torch.softmax(logits.float() + 1e9 * (col_mask.float() - 1.0)[:, None, None, :], dim=-1)
    weights = comm.all_gather(weights.contiguous(), 2)
    msa = msa + s * map_row_chunks(lambda part: ra._rows(part, weights), msa, ra.row_chunk)
    msa = msa + s * map_row_chunks(block.msa_transition, msa, block.msa_row_chunk)
    return msa, _pair_updates(block, z, mask_rows, mask_cols, comm, s, lambda t: t)


def _shard_rows(pair, comm: AxialComm):
    N = pair.shape[2]
    if N % comm.world:
        raise ValueError(f"axial sharding needs the token count ({N}) to be a multiple of the number of ranks ({comm.world})")
    return pair[:, comm.rows(N)].contiguous() if comm.world > 1 else pair


@torch.no_grad()
def sharded_pairformer_stack(blocks, pair, single, pair_mask, seq_mask, comm: AxialComm, gather: bool = True):
    """All ``blocks`` on row shards of the full pair tensor ``[B, N, N, C]`` (the same on every rank). With ``gather``
    the full pair tensor is reassembled on every rank at the end."""
    z = _shard_rows(pair, comm)
    for block in blocks:
        z, single = sharded_pairformer_block(block, z, single, pair_mask, seq_mask, comm)
    return (comm.all_gather(z, 1) if gather else z), single


@torch.no_grad()
def sharded_trunk(msa_blocks, pairformer_blocks, msa, pair, single, msa_mask, pair_mask, seq_mask, comm: AxialComm):
    """MSA stack then Pairformer stack of one trunk pass, the pair tensor sharded by rows from the first block to the
    last; returns ``(msa, pair, single)`` with the full pair tensor on every rank."""
    z = _shard_rows(pair, comm)
    for block in msa_blocks:
        msa, z = sharded_evoformer_block(block, msa, z, msa_mask, pair_mask, comm)
    for block in pairformer_blocks:
        z, single = sharded_pairformer_block(block, z, single, pair_mask, seq_mask, comm)
    return msa, comm.all_gather(z, 1), single
