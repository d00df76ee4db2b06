"""Multi-GPU forms of the operator path: one process per GPU, torch.distributed (NCCL) for the
few small exchanges the path needs. The reference is single-device; these have no counterpart
there and are checked against the single-device result.

* Row-sharded operators (RMSNorm, FusedAddRMSNorm, RoPE, SwiGLU, CrossEntropy, GRPO): tokens or
  sequences are split over ranks and every rank runs the ordinary operator on its rows. The only
  exchanges are: dW of the norms (sum all-reduce of [H]), the CE loss numerator and valid-row
  count, and the four GRPO reduction numerators.
* Vocab-parallel FusedLinearCrossEntropy: W is split by rows (vocabulary) over ranks, hidden and
  targets are replicated. Per row only (max, sum-exp, target logit) cross the wire, gathered in
  one all_gather of 3 floats per row; d(hidden) partial sums are then all-reduced once.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib as L
from ._lib import device_guard


# ------------------------------------------------------------------ partitioning (pure host logic)
def shard_bounds(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """[start, end) of rank's contiguous share of n items; shares are multiples of `multiple`
    except the last, differ by at most one multiple, and cover [0, n) exactly."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    units = -(-n // multiple)
    base, extra = divmod(units, world)
    start_u = rank * base + min(rank, extra)
    end_u = start_u + base + (1 if rank < extra else 0)
    return min(start_u * multiple, n), min(end_u * multiple, n)


def combine_rowstats(gathered: torch.Tensor) -> torch.Tensor:
    """gathered [G, 3, rows] of per-shard (max, sum exp(x - max), target logit) -> [3, rows] for the
    whole vocabulary: M = max_g m_g; S = sum_g s_g * exp(m_g - M); x_t = sum_g x_t,g (exactly one
    shard holds the target, the others contribute 0)."""
    m = gathered[:, 0]
    M = m.max(dim=0).values
    w = torch.exp(m - M)
    w = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(w), w)
    S = (gathered[:, 1] * w).sum(dim=0)
    xt = gathered[:, 2].sum(dim=0)
    return torch.stack([M, S, xt])


def _world(group):
    if not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


# ------------------------------------------------------------------ host-side failure detection
def check_vocab_sharding(BT: int, H: int, V_local: int, vocab_start: int, group=None) -> int:
    """Collective, host side, before anything is launched: every rank contributes (rows, hidden dim,
    shard height, shard start) and every rank checks the same list, so all of them accept or all of
    them raise ValueError. The shards must agree on rows and hidden dim and tile [0, V) without gap
    or overlap in rank order. Returns V. (A mismatch would otherwise show up as a collective on
    buffers of different sizes: a hang or a wrong loss.)"""
    world, rank = _world(group)
    mine = (int(BT), int(H), int(V_local), int(vocab_start))
    if world == 1:
        everyone = [mine]
    else:
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
    rows = {e[0] for e in everyone}
    dims = {e[1] for e in everyone}
    if len(rows) != 1 or len(dims) != 1:
        raise ValueError(f"vocab-parallel ranks disagree on hidden's shape (rows, hidden dim): {[(e[0], e[1]) for e in everyone]}")
    expect = 0
    for r, (_, _, v, start) in enumerate(everyone):
        if v <= 0 or start != expect:
            raise ValueError(f"vocabulary shards do not tile [0, V): rank {r} holds [{start}, {start + v}) but should start "
                             f"at {expect}; shards {[(e[3], e[3] + e[2]) for e in everyone]}")
        expect = start + v
    return expect


class RankWatch:
    """Liveness over the process group's key-value store, for the rule that a rank may leave only
    between steps with nothing of it in flight: the leaving rank calls ``leave()``; every other rank
    calls ``check()`` before it launches its next step and gets a RuntimeError naming the ranks that
    left, instead of entering a collective that can never complete. Pure host logic: no kernel and
    no collective is involved, so nothing has to time out on a GPU."""

    def __init__(self, store=None, rank=None, world=None, prefix="hilda_b200/left/"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix

    def leave(self, reason: str = "left") -> None:
        self.store.set(f"{self.prefix}{self.rank}", reason)

    def departed(self) -> list:
        return [r for r in range(self.world) if r != self.rank and self.store.check([f"{self.prefix}{r}"])]

    def check(self) -> None:
        gone = self.departed()
        if gone:
            raise RuntimeError(f"rank(s) {gone} left the job; not launching the next step")


# ------------------------------------------------------------------ row-sharded helpers
def allreduce_weight_grad(dW: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the norm weight gradient over row shards (in fp32, then back to dW's dtype)."""
    world, _ = _world(group)
    if world == 1:
        return dW
    buf = dW.float()
    dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    return buf.to(dW.dtype)


def rope_tables_for_sequence_shard(cos, sin, seq_local, rank=None, world=None, group=None):
    """RoPE with the SEQUENCE axis split over ranks (long context): rank r holds positions
    [r * seq_local, (r + 1) * seq_local), so it rotates with that slice of the half-width tables
    (..., seq_total, head_dim / 2). Returns views (no copy); the operator itself needs no exchange."""
    w, r = _world(group)
    world = w if world is None else world
    rank = r if rank is None else rank
    p0, p1 = rank * seq_local, (rank + 1) * seq_local
    if p1 > cos.shape[-2] or world * seq_local > cos.shape[-2]:
        raise ValueError(f"tables cover {cos.shape[-2]} positions, the {world} shards of {seq_local} need {world * seq_local}")
    return cos[..., p0:p1, :], sin[..., p0:p1, :]


def sharded_cross_entropy(logits_local, targets_local, ignore_index=-100, group=None):
    """Mean cross entropy over ALL ranks' rows; each rank holds a row shard. Returns (loss,
    dlogits_local). The valid-row count is all-reduced first (one int), so the kernel writes the
    gradient already scaled by the global 1/n_valid; the loss numerators are all-reduced after."""
    from .kernels.cross_entropy import cross_entropy_forward
    world, _ = _world(group)
    n_valid = (targets_local != ignore_index).sum(dtype=torch.int32)
    if world > 1:
        dist.all_reduce(n_valid, op=dist.ReduceOp.SUM, group=group)
    # 'mean' with the global count: loss_local = sum_local(loss rows) / n_valid_global
    loss, grad, _ = cross_entropy_forward(logits_local, targets_local, ignore_index, 'mean', needs_grad=True,
                                          n_valid_global=n_valid.reshape(1))
    if world > 1:
        loss = loss.clone()
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
    return loss, grad


def sharded_grpo_loss(logits_local, ids_local, adv_local, old_logp=None, ref_logp=None, mask_local=None,
                      temperature=1.0, beta=0.0, eps_low=0.2, eps_high=0.2, group=None):
    """GRPO loss over sequences sharded across ranks (equal sequences per rank). Returns
    (loss, kl_mean | None, clip_ratio, dlogits_local). The kernel normalises by the global number
    of sequences, so the only exchange is one all-reduce of four floats."""
    from .kernels.grpo_loss import grpo_loss_forward
    world, _ = _world(group)
    B = logits_local.shape[0]
    loss, kl_mean, clip, lse, mask, dlogits = grpo_loss_forward(
        logits_local, ids_local, adv_local, old_logp, ref_logp, mask_local, temperature, beta, eps_low, eps_high,
        needs_grad=True, batch_total=B * world)
    if world == 1:
        return loss, kl_mean, clip, dlogits
    msum = mask.sum()
    mden = msum.clamp(min=1.0)
    z = torch.zeros((), device=loss.device)
    vec = torch.stack([loss, (kl_mean * mden) if kl_mean is not None else z, clip * mden, msum])
    dist.all_reduce(vec, op=dist.ReduceOp.SUM, group=group)
    gden = vec[3].clamp(min=1.0)
    return vec[0], (vec[1] / gden) if kl_mean is not None else None, vec[2] / gden, dlogits


# ------------------------------------------------------------------ vocab-parallel FusedLinearCE
class VocabParallelFLCE:
    """Vocab-parallel fused linear + cross entropy. Every rank holds ``weight_shard`` = rows
    [vocab_start, vocab_start + V_local) of the lm_head and the full hidden / targets."""

    def __init__(self, group=None, comm_dtype=torch.float32, overlap_sms=0, validate=True):
        self.group = group
        # first call with a new (rows, hidden dim, shard height, shard start): one host-side collective
        # that checks the ranks' shards against each other (check_vocab_sharding); later calls skip it
        self.validate = validate
        self._validated = set()
        self.comm_dtype = comm_dtype  # dtype of the d(hidden) all-reduce
        # > 0: reduce each chunk's d(hidden) rows on a second stream beside that chunk's d(W) GEMM,
        # which then leaves this many SMs to the collective (needs comm_dtype == the data dtype)
        self.overlap_sms = int(overlap_sms)
        self.last_status = None
        self._side = {}
        self._reduce_group = None

    def _overlap_group(self):
        """Communicator of the overlapped d(hidden) all-reduce: a group of its own over the same ranks,
        so that the collective neither queues behind the row-statistics all-gathers of the main group
        nor ahead of them, with NCCL held to ``overlap_sms`` CTAs: the d(W) GEMM beside it leaves exactly
        that many SMs free, and a collective whose CTAs do not all fit waits for the GEMM to end
        instead of running beside it. Created on first use (a collective call: every rank gets here)."""
        if self._reduce_group is None:
            if dist.get_backend(self.group) != "nccl":
                self._reduce_group = self.group if self.group is not None else dist.group.WORLD
            else:
                ranks = dist.get_process_group_ranks(self.group if self.group is not None else dist.group.WORLD)
                opts = dist.ProcessGroupNCCL.Options()
                opts.config.max_ctas = max(1, self.overlap_sms)
                opts.config.min_ctas = 1
                # only the members of self.group get here: the new group is agreed among them alone
                self._reduce_group = dist.new_group(ranks, backend="nccl", pg_options=opts,
                                                    use_local_synchronization=True)
        return self._reduce_group

    def _side_stream(self, dev):
        key = torch.device(dev).index
        if key not in self._side:
            self._side[key] = torch.cuda.Stream(device=dev)
        return self._side[key]

    @staticmethod
    def _sm_count(dev):
        return torch.cuda.get_device_properties(dev).multi_processor_count

    def __call__(self, hidden, weight_shard, targets, vocab_start, ignore_index=-100, reduction='mean',
                 compute_grad=True, chunk_rows=None, skip_ignored=None):
        """Returns (loss, d_hidden, d_weight_shard). No host synchronisation: the count of non-ignored
        rows, the compaction of the ignored ones and the status word all stay on the device."""
        from .kernels import fused_linear_cross_entropy as FL
        if skip_ignored is None:
            skip_ignored = FL.SKIP_IGNORED_ROWS
        dev = L.require_cuda(hidden, weight_shard, targets)
        world, rank = _world(self.group)
        BT, H = hidden.shape
        V = weight_shard.shape[0]
        assert weight_shard.shape[1] == H and hidden.dtype == weight_shard.dtype
        assert hidden.dtype in (torch.bfloat16, torch.float16)
        assert targets.shape[0] == BT
        if self.validate and world > 1 and (BT, H, V, int(vocab_start)) not in self._validated:
            check_vocab_sharding(BT, H, V, int(vocab_start), self.group)
            self._validated.add((BT, H, V, int(vocab_start)))
        hidden = hidden.contiguous()
        weight_shard = weight_shard.contiguous()
        targets = targets.contiguous().long()
        dt = L.dt(hidden)
        esz = hidden.element_size()
        lib = L.lib()
        with device_guard(dev):
            st = L.stream(dev)
            if chunk_rows is None:
                chunk_rows = int(lib.hilda_flce_default_chunk_rows(BT, H, V))
            chunk_rows = max(1, min(chunk_rows, BT))
            n_chunks = -(-BT // chunk_rows)
            pitch, tiles = lib.hilda_flce_logits_pitch(V), lib.hilda_flce_stat_tiles(V)
            scratch = torch.empty(lib.hilda_flce_padded_rows(chunk_rows) * pitch, dtype=hidden.dtype, device=dev)
            stats = torch.empty(chunk_rows * tiles * 2, dtype=torch.float32, device=dev)
            rowstat = torch.empty(3, chunk_rows, dtype=torch.float32, device=dev)
            lse = torch.empty(chunk_rows, dtype=torch.float32, device=dev)
            loss_rows = torch.empty(BT, dtype=torch.float32, device=dev)
            head = torch.zeros(2, dtype=torch.int32, device=dev)  # [status, n_valid]
            status_p, n_valid_p = head.data_ptr(), head.data_ptr() + 4
            dyn = None
            h_use, t_use = hidden, targets
            if skip_ignored:
                # hidden and targets are replicated, so every rank drops the same ignored rows; the
                # lists are built on the device and every later step follows the device-side count
                idx = torch.empty(BT, dtype=torch.int64, device=dev)
                inv = torch.empty(BT, dtype=torch.int32, device=dev)
                t_use = torch.empty(BT, dtype=torch.int64, device=dev)
                h_use = torch.empty_like(hidden)
                L.check(lib.hilda_flce_compact(L.ptr(targets), BT, int(ignore_index), L.ptr(idx), L.ptr(inv),
                                               L.ptr(t_use), n_valid_p, st), "flce_compact")
                L.check(lib.hilda_gather_valid_rows(L.ptr(hidden), L.ptr(idx), n_valid_p, L.ptr(h_use), BT, H * esz, st),
                        "gather_valid_rows")
                dyn = n_valid_p
            else:
                L.check(lib.hilda_count_valid(L.ptr(targets), BT, int(ignore_index), n_valid_p, st), "count_valid")
            # partial sums of d(hidden) over the vocabulary shards: fp32 when they are reduced in fp32,
            # otherwise written by the GEMM directly in the 16-bit dtype they are reduced in
            reduce32 = compute_grad and world > 1 and self.comm_dtype == torch.float32
            dh32 = torch.empty(BT, H, dtype=torch.float32, device=dev) if reduce32 else None
            dh = torch.empty_like(hidden) if compute_grad else None
            dw = torch.empty_like(weight_shard) if compute_grad else None
            dw32 = torch.empty(V, H, dtype=torch.float32, device=dev) if (compute_grad and n_chunks > 1) else None
            if compute_grad and skip_ignored and world > 1:
                # rows of the compacted d(hidden) beyond the count are never written by the GEMM but
                # do take part in the all-reduce: they must hold finite values
                (dh32 if reduce32 else dh).zero_()
            reduced_rows = 0
            for c in range(n_chunks):
                r0 = c * chunk_rows
                rows = min(chunk_rows, BT - r0)
                hc = h_use[r0:r0 + rows]
                tc = t_use[r0:r0 + rows]
                L.check(lib.hilda_flce_logits(L.ptr(hc), L.ptr(weight_shard), L.ptr(scratch), L.ptr(stats), rows, H, V,
                                              dt, status_p, dyn, r0, st), "flce_logits")
                rs = rowstat[:, :rows].contiguous() if rows != chunk_rows else rowstat
                L.check(lib.hilda_flce_row_stats(L.ptr(stats), L.ptr(scratch), L.ptr(tc), L.ptr(rs), rows, V,
                                                 int(vocab_start), dt, dyn, r0, st), "flce_row_stats")
                n_shards = 1
                if world > 1:
                    gathered = torch.empty(world * 3, rows, dtype=torch.float32, device=dev)
                    dist.all_gather_into_tensor(gathered, rs, group=self.group)
                    rs, n_shards = gathered, world  # merged inside the finalize kernel
                L.check(lib.hilda_flce_finalize(L.ptr(rs), n_shards, L.ptr(tc), int(ignore_index), L.ptr(lse),
                                                loss_rows.data_ptr() + 4 * r0, rows, dyn, r0, st), "flce_finalize")
                if not compute_grad:
                    continue
                L.check(lib.hilda_flce_dlogits(L.ptr(scratch), L.ptr(lse), L.ptr(tc), int(ignore_index),
                                               n_valid_p if reduction == 'mean' else None, rows, V, int(vocab_start),
                                               dt, dyn, r0, st), "flce_dlogits")
                if reduce32:
                    L.check(lib.hilda_flce_grad_hidden(L.ptr(scratch), L.ptr(weight_shard), None,
                                                       dh32.data_ptr() + 4 * r0 * H, rows, H, V, dt, status_p, dyn, r0,
                                                       st), "flce_grad_hidden")
                else:
                    L.check(lib.hilda_flce_grad_hidden(L.ptr(scratch), L.ptr(weight_shard),
                                                       dh.data_ptr() + 2 * r0 * H, None, rows, H, V, dt, status_p, dyn,
                                                       r0, st), "flce_grad_hidden")
                mode = 3 if n_chunks == 1 else (0 if c == 0 else (2 if c == n_chunks - 1 else 1))
                overlap = world > 1 and self.overlap_sms > 0 and not reduce32 and self.comm_dtype == dh.dtype
                if overlap:
                    # this chunk's rows of d(hidden) are complete: reduce them over the ranks on a
                    # second stream while the d(W) GEMM runs here on all but `overlap_sms` SMs
                    side = self._side_stream(dev)
                    side.wait_stream(torch.cuda.current_stream(dev))
                    with torch.cuda.stream(side):
                        dist.all_reduce(dh[r0:r0 + rows], op=dist.ReduceOp.SUM, group=self._overlap_group())
                    lib.hilda_gemm_set_sm_limit(self._sm_count(dev) - self.overlap_sms)
                try:
                    L.check(lib.hilda_flce_grad_weight(L.ptr(scratch), L.ptr(hc), L.ptr(dw32), L.ptr(dw), mode, rows, H,
                                                       V, dt, status_p, dyn, r0, st), "flce_grad_weight")
                finally:
                    if overlap:
                        lib.hilda_gemm_set_sm_limit(0)
                if overlap:
                    reduced_rows = r0 + rows
            if compute_grad and world > 1 and reduced_rows == BT:
                torch.cuda.current_stream(dev).wait_stream(self._side_stream(dev))
            elif compute_grad and world > 1:
                if reduce32:
                    dist.all_reduce(dh32, op=dist.ReduceOp.SUM, group=self.group)
                    dh.copy_(dh32)
                elif self.comm_dtype == dh.dtype:
                    dist.all_reduce(dh, op=dist.ReduceOp.SUM, group=self.group)  # in place, no extra pass
                else:
                    buf = dh.to(self.comm_dtype)
                    dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
                    dh.copy_(buf)
            if skip_ignored:
                if compute_grad:
                    dh_c, dh = dh, torch.empty_like(hidden)
                    L.check(lib.hilda_scatter_valid_rows(L.ptr(dh_c), L.ptr(inv), L.ptr(dh), BT, H * esz, st),
                            "scatter_valid_rows")
                if reduction == 'none':
                    lr_c, loss_rows = loss_rows, torch.empty_like(loss_rows)
                    L.check(lib.hilda_scatter_valid_f32(L.ptr(lr_c), L.ptr(inv), L.ptr(loss_rows), BT, st),
                            "scatter_valid_f32")
            if reduction == 'none':
                loss = loss_rows
            else:
                # one reduction kernel; NaN if a bounded wait inside a GEMM ran out on this rank
                loss = torch.empty((), dtype=torch.float32, device=dev)
                L.check(lib.hilda_flce_sum_loss(L.ptr(loss_rows), BT, n_valid_p, 1 if reduction == 'mean' else 0,
                                                status_p, L.ptr(loss), st), "flce_sum_loss")
        self.last_status = head
        return loss, dh, dw

    def check_status(self):
        """Synchronises; raises if a device-side bounded wait ran out during the last call."""
        if self.last_status is not None and int(self.last_status[0]) != 0:
            raise RuntimeError(f"vocab-parallel FLCE: device status {int(self.last_status[0])}")
