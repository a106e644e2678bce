"""Tensor-parallel use of the path: KV heads are sharded over the ranks of one node and the
attention output is gathered along the last dimension before o_proj.

The reference expresses that gather as the `AllGatherDimLast` collective of its compiled schedule
(``src/bridge/segmented_runner.cpp:170-191``: an HCCL all-gather into scratch followed by a
transpose recipe).  Two forms are provided here, one process per GPU, `torch.distributed` (NCCL)
for the plumbing:

* ``mode="nccl"``  -- `all_gather_into_tensor` over NVLink/NVSwitch plus the rank-major -> last-dim
  permutation; the baseline.
* ``mode="push"``  -- the gather is fused into the attention epilogue: every rank's kernels store
  their ``[rows, cols]`` block straight into column block `rank` of every peer's gathered
  ``[rows, world*cols]`` buffer (plain peer stores into symmetric memory), followed by one small
  completion barrier with a bounded wait.  No collective kernel and no transpose run.

The gathered activation lives in a ring of `depth` buffers (2 by default): the buffer of exchange L
is written again by the peers at exchange L + depth, which they can start once the barrier of
exchange L + depth - 1 has let them pass, and that barrier needs this rank's arrival.  So whatever
reads exchange L's buffer on this rank (the next kernel of the stream, or a copy on a side stream)
has to be ordered before this rank's barrier of exchange L + depth - 1; a consumer on the same
stream is ordered automatically, a side-stream reader needs an event (`depth=3` gives it one whole
exchange of slack).  The barrier keeps its epoch in device memory, so a whole step (all layers)
can be captured in one CUDA graph and replayed; a captured step must contain a multiple of `depth`
exchanges so that every replay starts on the same buffer (`graph_safe`).

A bounded wait that runs out (a peer more than about a second late, or gone) does not raise by
itself: it sets GK_DEV_WAIT_EXPIRED in the device status word and the step goes on with whatever
arrived.  `check()` reads the word and raises; call it once per step, after the step's last
exchange, before the results are used.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    """Which heads a rank owns: rank r of `world` takes KV heads [r*Hkv/W, (r+1)*Hkv/W) and the query
    heads of those groups (the caller's column-parallel QKV projection already produces them)."""
    rank: int
    world: int
    q_heads: int
    kv_heads: int

    def __post_init__(self):
        if self.world <= 0 or not (0 <= self.rank < self.world):
            raise ValueError("GaudiRT: invalid tensor-parallel rank")
        if self.kv_heads % self.world or self.q_heads % self.kv_heads:
            raise ValueError("GaudiRT: KV heads must divide evenly over the tensor-parallel ranks")

    @property
    def local_kv_heads(self) -> int:
        return self.kv_heads // self.world

    @property
    def local_q_heads(self) -> int:
        return self.q_heads // self.world

    def kv_head_range(self):
        n = self.local_kv_heads
        return range(self.rank * n, (self.rank + 1) * n)

    def q_columns(self, head_dim: int) -> slice:
        n = self.local_q_heads * head_dim
        return slice(self.rank * n, (self.rank + 1) * n)

    def kv_columns(self, head_dim: int) -> slice:
        n = self.local_kv_heads * head_dim
        return slice(self.rank * n, (self.rank + 1) * n)


class OutputGather:
    """`[rows, cols]` per rank -> `[rows, world*cols]`, rank-major along the last dimension."""

    # bound of the completion wait in SM clock cycles (~1 s at 2 GHz); expiry sets a status bit
    WAIT_CYCLES = 2_000_000_000

    def __init__(self, rows: int, cols: int, device, group=None, mode: str = "push", depth: int = 2):
        if mode not in ("push", "nccl"):
            raise ValueError("GaudiRT: gather mode must be 'push' or 'nccl'")
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.rows, self.cols, self.mode, self.depth = rows, cols, mode, depth
        self.device = torch.device(device)
        self._turn = 0
        self._epoch = 0
        if mode == "nccl" or self.world == 1:
            self.mode = "nccl"
            self._staging = torch.empty(self.world, rows, cols, dtype=torch.bfloat16, device=self.device)
            return
        import torch.distributed._symmetric_memory as symm_mem
        width = self.world * cols
        self._local = symm_mem.empty(depth, rows, width, dtype=torch.bfloat16, device=self.device)
        self._flags = symm_mem.empty(max(self.world, 8), dtype=torch.int32, device=self.device)
        self._flags.zero_()
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)     # barrier epoch, kept on the device
        self._buf_handle = symm_mem.rendezvous(self._local, self.group)
        self._flag_handle = symm_mem.rendezvous(self._flags, self.group)
        block = slice(self.rank * cols, (self.rank + 1) * cols)
        self._peers = []            # [depth][peer] -> my column block of that peer's buffer
        for d in range(depth):
            per = []
            for p in range(self.world):
                buf = self._local if p == self.rank else self._buf_handle.get_buffer(
                    p, (depth, rows, width), torch.bfloat16)
                per.append(buf[d][:, block])
            self._peers.append(per)
        self._peer_flags = [self._flags if p == self.rank else
                            self._flag_handle.get_buffer(p, (self._flags.numel(),), torch.int32)
                            for p in range(self.world)]
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)          # every rank's flags are zero before anyone signals

    def graph_safe(self, exchanges_per_step: int) -> bool:
        """Whether a step of that many exchanges may be captured in a CUDA graph and replayed."""
        return self.mode == "nccl" or (exchanges_per_step % self.depth == 0 and self._turn % self.depth == 0)

    def destinations(self):
        """Tensors the attention epilogue of this step must write (push mode)."""
        return self._peers[self._turn % self.depth]

    def attention(self, query, key, value, key_pool, value_pool, metadata, head_dim, scale, softcap=0.0,
                  sliding_window=-1):
        """Paged attention on this rank's heads followed by the gather; returns `[rows, world*cols]`.
        With `key` and `value` None the step's rows are already in the pool (`_rotary_kv_store`)."""
        q_heads, kv_heads = query.size(1) // head_dim, key_pool.size(1)
        if self.mode == "nccl":
            if key is None:
                out = torch.ops.gaudirt._paged_attn_stored(query, key_pool, value_pool, metadata, head_dim, scale,
                                                           softcap, sliding_window)
            else:
                out = torch.ops.gaudirt.paged_attn(query, key, value, key_pool, value_pool, metadata, head_dim, scale,
                                                   softcap, sliding_window)
            return self.gather(out)
        plan = (metadata.attention_plan_for(q_heads, kv_heads, head_dim, sliding_window) if sliding_window > 0
                else metadata.attention_plan(q_heads, kv_heads, head_dim))
        torch.ops.gaudirt._paged_attn_push(query, key, value, key_pool, value_pool, metadata.row_locations(), plan,
                                           self.destinations(), head_dim, scale, softcap, sliding_window)
        return self.finish()

    def gather(self, out):
        """Baseline: NCCL all-gather + permutation of an already computed `[rows, cols]` block."""
        if self.world == 1:
            return out
        dist.all_gather_into_tensor(self._staging.view(self.world * self.rows, self.cols), out, group=self.group)
        return self._staging.permute(1, 0, 2).reshape(self.rows, self.world * self.cols)

    def finish(self):
        """Push mode: signal + bounded wait, then hand out the gathered buffer of this step."""
        torch.ops.gaudirt._peer_barrier_counted(self._peer_flags, self.rank, self._counter, self.WAIT_CYCLES)
        gathered = self._local[self._turn % self.depth]
        self._turn += 1
        return gathered

    def check(self):
        """Step-end check (synchronises): raises if a bounded wait ran out or a kernel met a bad slot or
        table entry during the step, instead of handing on an incomplete activation."""
        check_device_status(self.device)


_STATUS_TEXT = {1: "a slot outside the KV pool", 2: "a table entry outside the KV pool",
                4: "a bounded wait ran out (a peer is late or gone)", 8: "device-side metadata validation rejected a row"}


def check_device_status(device) -> None:
    """Reads and clears the status word of `device` and raises `RuntimeError` naming every bit set."""
    with torch.cuda.device(device):
        word = int(torch.ops.gaudirt._take_device_status())
    if word:
        what = "; ".join(text for bit, text in _STATUS_TEXT.items() if word & bit) or "unknown bits"
        raise RuntimeError(f"GaudiRT: device status {word} after the step: {what}")


class RowParallelOutput:
    """o_proj on this rank's heads, the rank-ordered sum of the partials, and the next layer's fused
    residual-add RMS norm (`O-Proj -> AllReduce -> AddRMSNorm`, the reference's usual tensor-parallel
    chain; sum semantics of ``src/bridge/communicator.cpp:373-417``: fp32 accumulator seeded with
    rank 0, ranks added in order, one rounding to bf16, so every rank holds the same bits).

    * ``mode="push"`` -- the tensor-core GEMM's epilogue stores its bf16 partial `[rows, hidden]` into
      slot `rank` of every peer's receive buffer (symmetric memory), one bounded completion barrier
      follows, and the sum is taken inside the norm kernel's prologue: no collective kernel runs and
      the summed activation is never written out.
    * ``mode="nccl"`` -- the baseline: local GEMM, `all_gather_into_tensor` of the partials, then the
      same rank-ordered sum + norm kernel (bit-identical by construction).
    """

    WAIT_CYCLES = OutputGather.WAIT_CYCLES

    def __init__(self, rows: int, hidden: int, device, group=None, mode: str = "push", depth: int = 2):
        if mode not in ("push", "nccl"):
            raise ValueError("GaudiRT: o_proj exchange mode must be 'push' or 'nccl'")
        if dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        else:                               # a single process: the sum has one term
            self.group, self.rank, self.world = None, 0, 1
        self.rows, self.hidden, self.mode, self.depth = rows, hidden, mode, depth
        self.device = torch.device(device)
        self._turn = 0
        self._epoch = 0
        if mode == "nccl" or self.world == 1:
            self.mode = "nccl"
            self._parts = torch.empty(self.world, rows, hidden, dtype=torch.bfloat16, device=self.device)
            return
        import torch.distributed._symmetric_memory as symm_mem
        shape = (depth, self.world, rows, hidden)
        self._local = symm_mem.empty(*shape, dtype=torch.bfloat16, device=self.device)
        self._flags = symm_mem.empty(max(self.world, 8), dtype=torch.int32, device=self.device)
        self._flags.zero_()
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._buf_handle = symm_mem.rendezvous(self._local, self.group)
        self._flag_handle = symm_mem.rendezvous(self._flags, self.group)
        self._peers = []            # [depth][peer] -> slot `rank` of that peer's receive buffer
        for d in range(depth):
            self._peers.append([(self._local if p == self.rank else
                                 self._buf_handle.get_buffer(p, shape, torch.bfloat16))[d][self.rank]
                                for p in range(self.world)])
        self._peer_flags = [self._flags if p == self.rank else
                            self._flag_handle.get_buffer(p, (self._flags.numel(),), torch.int32)
                            for p in range(self.world)]
        self._slots = [list(self._local[d].unbind(0)) for d in range(depth)]
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def partials(self, attn_out, weight):
        """This step's `[world, rows, hidden]` partials as a list of per-rank views, exchanged."""
        if self.mode == "nccl":
            return self.exchange(torch.ops.gaudirt._oproj(attn_out, weight))
        d = self._turn % self.depth
        torch.ops.gaudirt._oproj_push(attn_out, weight, self._peers[d])
        torch.ops.gaudirt._peer_barrier_counted(self._peer_flags, self.rank, self._counter, self.WAIT_CYCLES)
        self._turn += 1
        return self._slots[d]

    def graph_safe(self, exchanges_per_step: int) -> bool:
        """Whether a step of that many exchanges may be captured in a CUDA graph and replayed."""
        return self.mode == "nccl" or (exchanges_per_step % self.depth == 0 and self._turn % self.depth == 0)

    def check(self):
        """Step-end check (synchronises): raises if a bounded wait ran out during the step."""
        check_device_status(self.device)

    def exchange(self, mine):
        """Baseline exchange of an already computed `[rows, hidden]` partial: all-gather, rank-major."""
        if self.world == 1:
            return [mine]
        dist.all_gather_into_tensor(self._parts.view(self.world * self.rows, self.hidden), mine, group=self.group)
        return list(self._parts.unbind(0))

    def forward(self, attn_out, weight, residual, gamma, epsilon, weight_offset=0.0):
        """`attn_out [rows, local_heads*d]`, `weight [hidden, local_heads*d]` (this rank's columns of
        o_proj) -> `(normed, new_residual)` of the next layer, identical on every rank."""
        return torch.ops.gaudirt._rank_sum_add_rms_norm(self.partials(attn_out, weight), residual, gamma, epsilon,
                                                        weight_offset)

    def all_reduce(self, attn_out, weight):
        """o_proj followed by the plain rank-ordered sum (the all-reduced activation itself)."""
        return torch.ops.gaudirt._rank_sum(self.partials(attn_out, weight))
