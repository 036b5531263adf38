"""Single-rank step engine: owns weights, sequence state, row-bucketed step plans and CUDA graphs.

The reference builds one static Program per row bucket and optionally replays it from a HIP graph
(src/phaseshift/models/qwen35/runtime/executor.hip:806-823,991-1090).  Here a "program" is the Python
forward over fused kernels with stable workspace pointers; for decode-sized buckets it is captured
once into a CUDA graph and replayed, so a decode step costs one pinned H2D of the batch descriptor,
one graph launch and one 4-byte D2H per sampled row.

Step protocol (mirrors submit_co_batch / complete_batch, executor.hip:536-1132,2339-2423):
``reserve`` pages for every appended position -> run -> read status word -> ``commit`` positions, or
roll the reservation back and poison the sequences when the device reported a failure.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..utils.graphs import capture as capture_graph

from ..models.qwen35.config import Qwen35Config
from ..models.qwen35.model import Qwen35Runner, StepOutput
from ..models.qwen35.weights import EngineWeights, TpGeometry
from .batch import SeqRows, StepBatch, resolve_row_bucket
from .state import ModelState, StateConfig

GRAPH_MAX_ROWS = 8
GRAPH_MAX_DECODE_ROWS = 64      # pure decode batches (one row per sequence) are also replayed from graphs
GRAPH_MAX_VARIANT_ROWS = 16     # tapped / logged steps (speculative verification) replayed from graphs of their own


class SequenceError(RuntimeError):
    pass


@dataclass
class Sequence_:
    slot: int
    generation: int
    position: int = 0                   # committed tokens
    pages: List[int] = field(default_factory=list)
    poisoned: bool = False


class PageAllocator:
    """Slots and KV pages of the engine's own (non-batcher) sequences: a thin adapter over the host runtime's
    ``SlotPool`` / ``PagePool`` (csrc/runtime/runtime_core.cpp) -- the same free lists, generation counters and
    stale-handle check the serving batcher uses; page 0 stays reserved
    (reference: state/sequence_slot_pool.h:14-96, state/paged_kv_pool.h)."""

    def __init__(self, num_pages: int, max_slots: int):
        from ..core.native import runtime
        rt = runtime()
        self.slots, self.pages = rt.SlotPool(max_slots), rt.PagePool(num_pages)
        self.handles: Dict[int, object] = {}
        self.generation = [0] * max_slots

    def alloc_slot(self) -> Optional[int]:
        h = self.slots.acquire()
        if h.slot < 0:
            return None
        self.handles[h.slot] = h
        self.generation[h.slot] = h.generation
        return h.slot

    def release_slot(self, slot: int) -> None:
        self.slots.release(self.handles.pop(slot))      # raises on a stale handle
        self.generation[slot] += 1

    def alloc_page(self) -> Optional[int]:
        p = self.pages.acquire()
        return None if p < 0 else p

    def release_pages(self, pages: Sequence[int]) -> None:
        for p in pages:
            self.pages.release(int(p))

    @property
    def pages_free(self) -> int:
        return int(self.pages.free_count())


class Engine:
    def __init__(self, weights: EngineWeights, device, state_cfg: StateConfig, backend: str = "auto", tp=None,
                 use_graphs: bool = True, calibrate: bool = True, arena_gib: float = 0.0):
        """``calibrate``: fix the activation scales of the block-scaled tensor-core projections from one forward
        (once per weight set; see calibrate_act_scales)."""
        self.cfg: Qwen35Config = weights.cfg
        self.device = torch.device(device)
        if backend == "auto":
            backend = "cuda" if self.device.type == "cuda" else "ref"
        self.backend = backend
        geo = TpGeometry.make(self.cfg, weights.tp_rank, weights.tp_size)
        if backend == "cuda":
            from ..ops.cuda_ops import CudaOps
            self.ops = CudaOps(self.cfg, self.device, max_seq_len=state_cfg.max_seq_len)
        else:
            from ..ops.ref_ops import RefOps
            self.ops = RefOps(self.cfg, self.device)
        self.sc = state_cfg
        self.arenas = None
        if arena_gib and arena_gib > 0 and backend == "cuda":
            # KV pages and recurrent state live in virtual-memory arenas under this byte budget (`--arena-gib`)
            from ..core.arena import ArenaSet
            self.arenas = ArenaSet(int(arena_gib * (1 << 30)), self.device.index or 0)
        self.state = ModelState(self.cfg, state_cfg, self.device, self.ops.act_dtype, geo, arenas=self.arenas)
        self._arm_checked_limits()
        self.runner = Qwen35Runner(weights, self.state, self.ops, tp)
        self.tp = tp
        if tp is not None and hasattr(self.ops, "status"):
            tp.status_word = self.ops.status      # the transport's kernels report bounded-wait failures here
        self.alloc = PageAllocator(self.state.num_pages, state_cfg.max_slots)
        self.seqs: Dict[int, Sequence_] = {}
        self.batches: Dict[int, StepBatch] = {}
        self.graphs: Dict[int, object] = {}
        self.graph_out: Dict[int, StepOutput] = {}
        self.launches_per_graph: Dict[int, int] = {}
        self.use_graphs = use_graphs and backend == "cuda"
        if tp is not None and tp.size > 1 and tp.transport != "fused":
            # the library all-reduce is not captured into CUDA graphs; only the in-kernel combine is
            self.use_graphs = False
        if tp is not None and tp.size > 1 and backend == "cuda":
            # transport self-test + the collective allocations, before the first real step; a failed test drops
            # every rank to the library transport (which is not graph-captured)
            tp.status_word = self.ops.status
            if not tp.verify(self.ops):
                self.use_graphs = False
        self.h_tokens = torch.zeros(2048, dtype=torch.int32, pin_memory=(self.device.type == "cuda"))
        self.h_status = torch.zeros(2, dtype=torch.int32, pin_memory=(self.device.type == "cuda"))
        self.h_extra = torch.zeros(64, dtype=torch.int32, pin_memory=(self.device.type == "cuda"))
        self._h_pages = torch.zeros(64, max(64, self.state.max_blocks), dtype=torch.int32, pin_memory=(self.device.type == "cuda"))
        self._h_pages_next = 0
        self.graph_variants = True      # verification / tapped steps replay captured graphs too
        # greedy, unmasked steps whose logits nobody asked for sample inside the lm_head kernel (PS_FUSED_ARGMAX=0: never)
        self.fused_argmax = self.backend == "cuda" and os.environ.get("PS_FUSED_ARGMAX", "1") != "0"
        self.graph_refs: Dict[object, object] = {}
        self.steps = 0
        self.status_errors = 0
        self.act_scales_calibrated = False
        # once per weight set: a second engine over the same weights must run the same arithmetic as the first
        if (calibrate and backend == "cuda" and getattr(weights, "layout", "") in ("tc", "both")
                and not getattr(weights, "act_scales_calibrated", False)):
            self.calibrate_act_scales()
            weights.act_scales_calibrated = True
        if tp is not None and tp.size > 1 and backend == "cuda":
            self._tp_warmup()

    def _raise_if_peer_lost(self, e: BaseException) -> None:
        """A library collective that failed under tensor parallelism (connection closed by a peer that exited, process
        group timeout) means a rank is gone: surface it as RankLostError, naming the ranks once the heartbeat knows."""
        if self.tp is None or self.tp.size <= 1:
            return
        msg = str(e)
        if not any(k in msg for k in ("Connection closed", "Connection reset", "timed out", "Timed out", "timeout", "NCCL",
                                      "gloo", "ProcessGroup", "Broken pipe")):
            return
        import time
        from ..parallel.health import RankLostError
        mon = getattr(self.tp, "monitor", None)
        lost: List[int] = []
        if mon is not None:
            deadline = time.monotonic() + mon.timeout_s + 4 * mon.interval_s
            while not lost and time.monotonic() < deadline:
                lost = mon.lost()
                if not lost:
                    time.sleep(mon.interval_s)
        raise RankLostError(lost) from e

    def _tp_warmup(self) -> None:
        """Tensor parallel: everything a first step would do lazily -- weight tiling, kernel attributes, symmetric
        buffers of the combine / scatter paths -- happens here on every rank, followed by a barrier, so the ranks enter
        their first real step together instead of skewed by seconds of one-off host work (device waits are bounded)."""
        import torch.distributed as dist
        graphs, self.use_graphs = self.use_graphs, False
        s = self.open_sequence()
        try:
            n = max(1, min(40, self.sc.max_seq_len - 2))
            self.step([SeqRows(s.slot, 0, [1] * n, (n - 1,))], [s])
            self.step([SeqRows(s.slot, s.position, [1], (0,))], [s])
        finally:
            self.close_sequence(s)
            self.use_graphs = graphs
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(self.tp.group)
        self.steps = 0

    def set_uniform_arithmetic(self, on: bool) -> None:
        """Speculative decoding needs every step of a sequence -- single-row decode, multi-row verification, the
        plain fallback rounds -- on one projection arithmetic, or verified tokens would not reproduce plain decoding
        (the reference's Exact verify mode, include/phaseshift/runtime/execution/execution_types.h:6-27).  With both
        weight layouts resident single-row steps normally stream with bf16 activations; this pins them to the
        tensor-core kernel that multi-row steps use.  Captured graphs are dropped because they bake the choice in."""
        if hasattr(self.ops, "force_tc") and self.ops.force_tc != on:
            self.ops.force_tc = on
            self.graphs.clear()
            self.graph_out.clear()
            self.graph_refs.clear()
            self.launches_per_graph.clear()

    # ------------------------------------------------------------------ activation scales (tensor-core layout)
    def calibrate_act_scales(self, token_ids: Optional[Sequence[int]] = None, n_tokens: int = 64) -> Dict[str, float]:
        """Fix the NVFP4 activation scale of every projection input site from one forward over `token_ids`
        (default: `n_tokens` pseudo-random ids): the largest |x| seen at the site maps to a block scale of 32, which
        leaves 14x of headroom before the UE4M3 block scale saturates and 11 binades below it at full precision.
        The reference's activation quantiser scales each row by its own maximum
        (src/phaseshift/models/qwen35/kernels/optimized/activation_quantize.hip:65-120); a fixed scale lets the
        projection kernel quantise K-panels independently inside its prologue.  Every rank calibrates its own slice."""
        from ..quant.act_quant import calibrate_act_scale
        from ..models.qwen35.weights import P as _P
        w = self.runner.w
        sites: Dict[str, object] = {_P + "lm_head.weight": w.lm_head}
        for li, L in enumerate(w.layers):
            lp = f"{_P}layers.{li}."
            m = L.mixer
            if L.kind == 0:
                sites[lp + "linear_attn.in_proj_qkv.weight"] = m.in_proj
                sites[lp + "linear_attn.out_proj.weight"] = m.out_proj
            else:
                sites[lp + "self_attn.q_proj.weight"] = m.qkv_proj
                sites[lp + "self_attn.o_proj.weight"] = m.o_proj
            sites[lp + "mlp.gate_proj.weight"] = L.gate_up
            sites[lp + "mlp.down_proj.weight"] = L.down
        if token_ids is None:
            g = torch.Generator().manual_seed(20240229)
            n = max(1, min(n_tokens, self.sc.max_seq_len - 1))
            token_ids = torch.randint(0, self.cfg.vocab_size, (n,), generator=g).tolist()
        seen: Dict[str, torch.Tensor] = {}

        def collect(tag: str, x: torch.Tensor) -> None:
            a = x.detach().abs().amax().float()
            seen[tag] = a if tag not in seen else torch.maximum(seen[tag], a)

        prev = self.runner.act_collector
        self.runner.act_collector = collect
        graphs = self.use_graphs
        self.use_graphs = False
        s = self.open_sequence()
        try:
            with torch.no_grad():
                r = SeqRows(s.slot, 0, list(token_ids), output_rows=(len(token_ids) - 1,))
                self.step([r], [s])
        finally:
            self.close_sequence(s)
            self.runner.act_collector = prev
            self.use_graphs = graphs
        out = {}
        for tag, a in seen.items():
            W = sites.get(tag)
            if W is not None and W.fmt == "nvfp4":
                W.act_scale = calibrate_act_scale(float(a))
                out[tag] = W.act_scale
        self.act_scales_calibrated = True
        return out

    # ------------------------------------------------------------------ sequences
    def open_sequence(self) -> Sequence_:
        slot = self.alloc.alloc_slot()
        if slot is None:
            raise SequenceError("no free sequence slot")
        s = Sequence_(slot, self.alloc.generation[slot])
        self.state.reset_slot(slot)
        self.state.block_table[slot].fill_(-1)
        self.seqs[slot] = s
        return s

    def close_sequence(self, s: Sequence_) -> None:
        if self.alloc.generation[s.slot] != s.generation:
            raise SequenceError("stale sequence handle")
        self.alloc.release_pages(s.pages)
        s.pages = []
        self.alloc.release_slot(s.slot)
        del self.seqs[s.slot]

    def _reserve(self, s: Sequence_, upto: int) -> int:
        """Map pages so positions < upto exist; returns how many pages were added (for rollback)."""
        pt = self.sc.page_tokens
        need = -(-upto // pt)
        if need > self.state.max_blocks:
            raise SequenceError("sequence exceeds max_seq_len")
        added = 0
        new_entries = []
        while len(s.pages) < need:
            pg = self.alloc.alloc_page()
            if pg is None:
                self.alloc.release_pages(s.pages[len(s.pages) - added:])
                del s.pages[len(s.pages) - added:]
                raise SequenceError("out of KV pages")
            new_entries.append((len(s.pages), pg))
            s.pages.append(pg)
            added += 1
        if new_entries:
            idx0, n = new_entries[0][0], len(new_entries)
            if self.device.type == "cuda":
                # pinned staging ring: no pageable (synchronous) host-to-device copy on the step path; a region is
                # reused only after `_h_pages_slots` further reservations, by which time its copy has long been issued
                # and consumed in stream order
                if n > self._h_pages.shape[1]:
                    self._h_pages = torch.zeros(self._h_pages.shape[0], n, dtype=torch.int32, pin_memory=True)
                row = self._h_pages[self._h_pages_next % self._h_pages.shape[0]]
                self._h_pages_next += 1
                if self._h_pages_next % self._h_pages.shape[0] == 0:
                    torch.cuda.current_stream().synchronize()      # once per ring cycle: every staged copy has landed
                row[:n] = torch.as_tensor([p for _, p in new_entries], dtype=torch.int32)
                self.state.block_table[s.slot, idx0:idx0 + n].copy_(row[:n], non_blocking=True)
            else:
                self.state.block_table[s.slot, idx0:idx0 + n] = torch.tensor([p for _, p in new_entries], dtype=torch.int32)
        return added

    def trim_pages(self, s: Sequence_) -> None:
        """Return pages past the committed position (after a speculative step kept fewer rows)."""
        pt = self.sc.page_tokens
        need = -(-max(s.position, 1) // pt)
        if len(s.pages) > need:
            extra = s.pages[need:]
            del s.pages[need:]
            self.state.block_table[s.slot, need:need + len(extra)] = -1
            self.alloc.release_pages(extra)

    # ------------------------------------------------------------------ stepping
    def _batch(self, bucket: int) -> StepBatch:
        b = self.batches.get(bucket)
        if b is None:
            b = StepBatch(bucket, min(bucket, self.sc.max_slots), self.device)
            b.max_context = self.sc.max_seq_len + 1
            self.batches[bucket] = b
        return b

    def step(self, rows: Sequence[SeqRows], seq_objs: Sequence[Sequence_], *, commit: bool = True,
             tap_layers: Sequence[int] = (), gdn_log=None, gdn_to_alt: bool = False, mask=None,
             mask_active=None, want_logits: bool = False, sample: bool = True, exact: bool = False,
             device_ids=None, read_back: Optional[torch.Tensor] = None):
        """Run one step.  Returns (tokens list[int] per output row, StepOutput).

        ``device_ids`` = (first row, int32 device tensor): token ids of those rows are taken from the device tensor
        instead of ``rows`` (speculative drafts that were never read back); ``read_back``: a small int32 device tensor
        copied to the host together with the sampled tokens (``StepOutput.read_back``), so that the step stays the
        round's only host synchronisation.

        ``exact``: compute every row with single-row-decode arithmetic (the reference's VerifyNumericMode::Exact,
        include/phaseshift/runtime/execution/execution_types.h:6-27): projections stay on the batch-invariant
        small-M kernel instead of the tensor-core GEMM, so speculative verification reproduces plain decoding."""
        if self.tp is not None:
            self.tp.assert_alive()           # host-side heartbeat: never launch towards a peer that is gone
        n_rows = sum(len(r.token_ids) for r in rows)
        n_out = sum(len(r.output_rows) for r in rows)
        bucket = resolve_row_bucket(n_rows)
        b = self._batch(bucket)
        added = []
        try:
            for r, s in zip(rows, seq_objs):
                if s.poisoned:
                    raise SequenceError("sequence is poisoned")
                if r.pos_start != s.position and commit:
                    raise SequenceError("rows must start at the committed position")
                added.append(self._reserve(s, r.pos_start + len(r.token_ids)))
        except SequenceError:
            for s, a in zip(seq_objs, added):
                if a:
                    self.alloc.release_pages(s.pages[-a:])
                    del s.pages[-a:]
            raise
        try:
            toks, out, status = self._execute(rows, n_rows, n_out, bucket, b, tap_layers=tap_layers, gdn_log=gdn_log,
                                              gdn_to_alt=gdn_to_alt, mask=mask, mask_active=mask_active, sample=sample,
                                              exact=exact, device_ids=device_ids, read_back=read_back, want_logits=want_logits)
        except RuntimeError as e:
            self._raise_if_peer_lost(e)
            raise
        if status != 0:
            for s in seq_objs:
                s.poisoned = True
            raise SequenceError(f"device reported status {status}; sequences poisoned")
        if commit:
            for r, s in zip(rows, seq_objs):
                s.position = r.pos_start + len(r.token_ids)
        return toks, out

    GREEDY_KEY_BIT = 1 << 48

    @classmethod
    def graph_key(cls, bucket: int, n_out: int, identity_out: bool, greedy: bool = False) -> int:
        """Key of a plain captured step in ``graphs`` / ``graph_out`` / ``launches_per_graph`` (variants wrap it in a tuple)."""
        return ((bucket * 4096 + n_out) * 2 + (1 if identity_out else 0)) | (cls.GREEDY_KEY_BIT if greedy else 0)

    @classmethod
    def graph_key_bucket(cls, key) -> int:
        k = key[0] if isinstance(key, tuple) else key
        return ((k & (cls.GREEDY_KEY_BIT - 1)) // 2) // 4096

    def _arm_checked_limits(self) -> None:
        """Checked library: the descriptor limits and the status word its assertions report to live in one device symbol per
        kernel file, shared by every engine of the process, so each engine registers its own before it launches (a second
        engine with fewer slots would otherwise make the first one's kernels skip its higher slots, silently for it)."""
        if getattr(self.ops, "checked", False):
            from ..ops import _lib as _klib
            _klib.set_limits(self.sc.max_slots, 1 << 20, self.state.status)

    def _run_graph(self, bucket: int, b: StepBatch, n_out: int, variant=None, greedy: bool = False) -> StepOutput:
        """``variant`` = (tap layers, GDN log dict or None, to_alt, exact): steps that tap hidden states or log the
        recurrent updates get graphs of their own (the tap and log tensors are fixed buffers, so the capture stays
        valid; Exact mode only changes which kernels the host picks, which the capture bakes in)."""
        key = self.graph_key(bucket, n_out, b.identity_out, greedy)
        kw = {}
        if variant is not None:
            taps, log, to_alt, exact = variant
            key = (key, tuple(taps), id(log) if log is not None else 0, to_alt, exact)
            kw = dict(tap_layers=taps, gdn_log=log, gdn_to_alt=to_alt)
        if greedy:
            kw["greedy_only"] = True          # a graph of its own: the sampling kernel is not in it
        g = self.graphs.get(key)
        if g is None:
            self.ops.exact_rows = bool(variant[3]) if variant is not None else False
            try:
                # warm up once outside capture (allocates workspaces, sets kernel attributes)
                self.runner.forward(b, bucket, n_out, **kw)
                torch.cuda.current_stream().synchronize()
                l0 = self.ops.launches
                g, out = capture_graph(self.device, lambda: self.runner.forward(b, bucket, n_out, **kw))
            finally:
                self.ops.exact_rows = False
            if variant is not None:
                self.graph_refs[key] = variant[1]          # keeps the log tensors (and the id in the key) alive
            self.launches_per_graph[key] = self.ops.launches - l0
            self.graphs[key] = g
            self.graph_out[key] = out
            # the warm-up and capture forwards ran the real step already (state was updated once by the
            # warm-up, capture does not execute), so fall through to a replay only on later calls
            return self._replay_after_warmup(key)
        g.replay()
        return self.graph_out[key]

    def _replay_after_warmup(self, key: int) -> StepOutput:
        # The warm-up forward already produced this step's results in the same workspace buffers.
        return self.graph_out[key]

    # ------------------------------------------------------------------ externally managed sequences
    def apply_block_updates(self, updates) -> None:
        """Write (slot, block, page) entries produced by the host runtime into the device block table."""
        if not updates:
            return
        u = torch.tensor(updates, dtype=torch.int64)
        bt = self.state.block_table
        vals = u[:, 2].to(torch.int32)
        if self.device.type == "cuda":
            bt.index_put_((u[:, 0].to(self.device), u[:, 1].to(self.device)), vals.to(self.device))
        else:
            bt[u[:, 0], u[:, 1]] = vals

    def run_rows(self, rows: Sequence[SeqRows], *, mask=None, mask_active=None, tap_layers: Sequence[int] = (),
                 gdn_log=None, gdn_to_alt: bool = False, sample: bool = True, want_logits: bool = False):
        """Execute one step for sequences whose slots/pages are managed by the caller (the batcher).
        Returns (tokens, StepOutput, device_status)."""
        if self.tp is not None:
            self.tp.assert_alive()
        n_rows = sum(len(r.token_ids) for r in rows)
        n_out = sum(len(r.output_rows) for r in rows)
        bucket = resolve_row_bucket(n_rows)
        b = self._batch(bucket)
        try:
            return self._execute(rows, n_rows, n_out, bucket, b, tap_layers=tap_layers, gdn_log=gdn_log,
                                 gdn_to_alt=gdn_to_alt, mask=mask, mask_active=mask_active, sample=sample, exact=False,
                                 want_logits=want_logits)
        except RuntimeError as e:
            self._raise_if_peer_lost(e)
            raise

    def _execute(self, rows, n_rows: int, n_out: int, bucket: int, b: StepBatch, *, tap_layers, gdn_log, gdn_to_alt,
                 mask, mask_active, sample: bool, exact: bool, device_ids=None, read_back=None, want_logits: bool = False):
        """Fill and upload the batch descriptor, run the forward (graph replay for plain decode-sized steps, eager
        otherwise), read back sampled ids and every device status word with one stream synchronisation.  Returns
        (tokens, StepOutput, status); a non-zero status has already been cleared on the device (together with any
        stream-K flags a kernel that gave up may have left raised) and it is the caller's job to poison sequences.
        Status words: the state's own (bad page / slot indices), the op set's (bounded waits of the projection and
        all-reduce kernels; the tensor-parallel transport writes into the same word)."""
        self._arm_checked_limits()
        b.fill(rows)
        # every output row greedy, unmasked, and the logits of no interest: the lm_head samples in its own epilogue
        greedy = (self.fused_argmax and sample and mask is None and not want_logits and not exact and n_out > 0
                  and all(r.temperature <= 0.0 for r in rows))
        plain = not tap_layers and gdn_log is None and not gdn_to_alt and mask is None and sample and not exact
        decode_batch = bucket <= GRAPH_MAX_DECODE_ROWS and all(len(r.token_ids) == 1 for r in rows)
        use_graph = self.use_graphs and plain and (bucket <= GRAPH_MAX_ROWS or decode_batch)
        # tapped / logged / Exact steps (speculative verification, tapped decode): graphs of their own
        variant = None
        if (self.use_graphs and self.graph_variants and not plain and mask is None and sample
                and bucket <= GRAPH_MAX_VARIANT_ROWS):
            variant = (tuple(tap_layers), gdn_log, bool(gdn_to_alt), bool(exact))
            use_graph = True
        b.graph_static = use_graph
        b.upload()
        if device_ids is not None:
            r0, t = device_ids
            b.ids[r0:r0 + t.numel()].copy_(t, non_blocking=True)
        if use_graph:
            out = self._run_graph(bucket, b, n_out, variant, greedy)
        else:
            self.ops.exact_rows = exact
            try:
                out = self.runner.forward(b, bucket if self.backend == "cuda" else n_rows, n_out, tap_layers=tap_layers,
                                          gdn_log=gdn_log, gdn_to_alt=gdn_to_alt, mask=mask, mask_active=mask_active,
                                          sample=sample, **({"greedy_only": True} if greedy else {}))
            finally:
                self.ops.exact_rows = False
        toks: List[int] = []
        ops_status = getattr(self.ops, "status", None)
        if self.device.type == "cuda":
            if out.tokens is not None and n_out:
                self.h_tokens[:n_out].copy_(out.tokens[:n_out], non_blocking=True)
            self.h_status[0:1].copy_(self.state.status, non_blocking=True)
            if ops_status is not None:
                self.h_status[1:2].copy_(ops_status, non_blocking=True)
            if read_back is not None:
                self.h_extra[:read_back.numel()].copy_(read_back, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            if read_back is not None:
                out.read_back = self.h_extra[:read_back.numel()].tolist()
            status = int(self.h_status[0]) or int(self.h_status[1])
            if out.tokens is not None:
                toks = self.h_tokens[:n_out].tolist()
        else:
            status = int(self.state.status[0])
            if status == 0 and ops_status is not None:
                status = int(ops_status[0])
            if out.tokens is not None:
                toks = out.tokens[:n_out].tolist()
            if read_back is not None:
                out.read_back = read_back.tolist()
        self.steps += 1
        if getattr(self.ops, "checked", False):
            # checked mode also looks at the step's hidden rows: the block-scaled projections quantise their inputs, which
            # turns a NaN from further up into finite codes, so a fault can pass the logits unseen on the tensor-core path
            if out.hidden is not None and n_out and not bool(torch.isfinite(out.hidden[:n_out].float()).all()):
                raise RuntimeError("checked build: non-finite hidden states at the output rows of this step")
            bad = self.ops.check_canaries()
            if bad:
                raise RuntimeError("checked build: workspace guard bytes overwritten around " + ", ".join(sorted(set(bad))))
        if status != 0:
            self.status_errors += 1
            self.state.status.zero_()
            if ops_status is not None:
                ops_status.zero_()
            if hasattr(self.ops, "reset_after_error"):
                self.ops.reset_after_error()
        return toks, out, status

    def profile_step(self, rows: Sequence[SeqRows], seq_objs: Sequence[Sequence_], **kw) -> Dict[str, dict]:
        """Run one step eagerly with per-op-family device timing (ops/trace.py).  Returns name -> {calls, ms}; the
        step itself behaves like ``step(..., commit=False)`` unless told otherwise."""
        graphs, self.use_graphs = self.use_graphs, False
        self.ops.collect_times()
        self.ops.op_times = {}
        self.ops.timing_enabled = True
        try:
            kw.setdefault("commit", False)
            self.step(rows, seq_objs, **kw)
        finally:
            self.ops.timing_enabled = False
            self.use_graphs = graphs
        t = self.ops.collect_times()
        return {k: {"calls": v[0], "ms": round(v[1], 4)} for k, v in sorted(t.items(), key=lambda kv: -kv[1][1])}

    # ------------------------------------------------------------------ convenience: one request
    def prefill(self, s: Sequence_, token_ids: Sequence[int], chunk: int = 2048, sample_last: bool = True,
                **samp) -> Optional[int]:
        tok = None
        n = len(token_ids)
        for c0 in range(0, n, chunk):
            ids = token_ids[c0:c0 + chunk]
            last = c0 + chunk >= n
            r = SeqRows(s.slot, s.position, ids, output_rows=(len(ids) - 1,) if (last and sample_last) else (), **samp)
            toks, _ = self.step([r], [s])
            if toks:
                tok = toks[0]
        return tok

    def decode(self, s: Sequence_, token: int, **samp) -> int:
        r = SeqRows(s.slot, s.position, [token], output_rows=(0,), **samp)
        toks, _ = self.step([r], [s])
        return toks[0]

    def generate(self, prompt: Sequence[int], max_new_tokens: int, prefill_chunk: int = 2048, temperature: float = 0.0,
                 top_p: float = 1.0, top_k: int = 0, seed: int = 0, eos: Sequence[int] = ()) -> List[int]:
        s = self.open_sequence()
        try:
            out: List[int] = []
            samp = dict(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed)
            tok = self.prefill(s, prompt, prefill_chunk, sample_index=0, **samp)
            out.append(tok)
            while len(out) < max_new_tokens and tok not in eos:
                tok = self.decode(s, tok, sample_index=len(out), **samp)
                out.append(tok)
            return out
        finally:
            self.close_sequence(s)
