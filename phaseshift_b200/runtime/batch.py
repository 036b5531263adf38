"""Per-step batch descriptor (the analogue of the reference's DeviceBatchContext,
include/phaseshift/runtime/batch/device_batch_context.h:14-85).

The host describes a step by *requests* (slot, first position, number of rows, which rows need logits);
the per-row arrays the kernels index (token id, slot, position) are expanded into ONE packed int32
buffer that goes to the device with ONE pinned host-to-device copy.  The device buffers are allocated
once per row bucket, so a captured CUDA graph can be replayed after refreshing them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

ROW_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048)


def resolve_row_bucket(rows: int) -> int:
    """Smallest bucket holding `rows` (reference: include/phaseshift/runtime/execution/row_bucket.h:7-68,
    extended downwards: on B200 decode steps are graph-captured per small bucket)."""
    for b in ROW_BUCKETS:
        if rows <= b:
            return b
    raise ValueError(f"{rows} rows exceed the largest row bucket {ROW_BUCKETS[-1]}")


@dataclass
class SeqRows:
    slot: int
    pos_start: int
    token_ids: Sequence[int]
    output_rows: Sequence[int] = ()        # indices into token_ids whose logits are sampled
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = 0
    sample_index: int = 0                  # tokens generated so far (first output row); +1 per further row


SAMPLING_ROW_DTYPE = np.dtype([("mode", "<u4"), ("temperature", "<f4"), ("top_p", "<f4"), ("top_k", "<u4"),
                               ("seed", "<u8"), ("sample_index", "<u8")])


class StepBatch:
    """Host-side packed step + its device mirror."""
    SHORT_SEQ_ROWS = 16          # = CudaOps.ATTN_PREFILL_MIN_ROWS: sequences with more rows take the tiled attention kernel

    def __init__(self, max_rows: int, max_seqs: int, device, pinned: Optional[bool] = None):
        self.max_rows, self.max_seqs, self.device = max_rows, max_seqs, device
        use_pin = (device.type == "cuda") if pinned is None else pinned
        n_int = 3 * max_rows + 4 * max_seqs + 2 * max_rows    # ids, slot, pos | seq descs | output rows | pos of short sequences' rows
        self.h_int = torch.zeros(n_int, dtype=torch.int32, pin_memory=use_pin)
        self.h_samp = torch.zeros(max_rows * SAMPLING_ROW_DTYPE.itemsize, dtype=torch.uint8, pin_memory=use_pin)
        self.d_int = torch.zeros(n_int, dtype=torch.int32, device=device)
        self.d_samp = torch.zeros_like(self.h_samp, device=device)
        self.n_rows = self.n_seqs = self.n_out = 0
        self.max_visible = 1
        # graph_static: the step is replayed from a captured CUDA graph, so launch geometry must not
        # depend on this step's contents (attention covers max_context, GDN covers max_seqs descriptors)
        self.graph_static = False
        self.identity_out = False
        self.max_context = 1
        o = 0
        self.ids = self.d_int[o:o + max_rows]; o += max_rows
        self.row_slot = self.d_int[o:o + max_rows]; o += max_rows
        self.row_pos = self.d_int[o:o + max_rows]; o += max_rows
        self.seq_desc = self.d_int[o:o + 4 * max_seqs].view(max_seqs, 4); o += 4 * max_seqs
        self.out_rows = self.d_int[o:o + max_rows]; o += max_rows
        # positions of the rows of sequences with at most SHORT_SEQ_ROWS rows in the step, -2 for the rows of longer sequences
        # (the per-row attention kernel leaves those rows' outputs alone: the tiled kernel of the same step wrote them) and
        # -1 for padding rows
        self.row_pos_short = self.d_int[o:o + max_rows]
        self._np = self.h_int.numpy()
        self._np_samp = self.h_samp.numpy().view(SAMPLING_ROW_DTYPE)
        self.seqs: List[SeqRows] = []

    def fill(self, seqs: Sequence[SeqRows]) -> None:
        mr, ms = self.max_rows, self.max_seqs
        a = self._np
        a[:] = 0
        a[mr:3 * mr] = -1          # padding rows of a bucket: slot -1 / position -1, skipped by the kernels
        short0 = 3 * mr + 4 * ms + mr
        a[short0:short0 + mr] = -1
        r = 0
        n_out = 0
        max_vis = 1
        if len(seqs) > ms:
            raise ValueError("too many sequences for this batch")
        for i, s in enumerate(seqs):
            n = len(s.token_ids)
            if r + n > mr:
                raise ValueError("too many rows for this batch")
            a[r:r + n] = np.asarray(s.token_ids, dtype=np.int32)
            a[mr + r:mr + r + n] = s.slot
            a[2 * mr + r:2 * mr + r + n] = np.arange(s.pos_start, s.pos_start + n, dtype=np.int32)
            a[short0 + r:short0 + r + n] = a[2 * mr + r:2 * mr + r + n] if n <= self.SHORT_SEQ_ROWS else -2
            a[3 * mr + 4 * i:3 * mr + 4 * i + 4] = (r, n, s.slot, s.pos_start)
            for j, orow in enumerate(s.output_rows):
                a[3 * mr + 4 * ms + n_out] = r + orow
                sp = self._np_samp[n_out]
                sp["mode"] = 1 if s.temperature <= 0.0 else 2
                sp["temperature"], sp["top_p"], sp["top_k"] = s.temperature, s.top_p, s.top_k
                sp["seed"], sp["sample_index"] = s.seed, s.sample_index + j
                n_out += 1
            max_vis = max(max_vis, s.pos_start + n)
            r += n
        self.n_rows, self.n_seqs, self.n_out, self.max_visible = r, len(seqs), n_out, max_vis
        # output row i is step row i for every i (a pure decode batch): the output gather is the identity
        self.identity_out = n_out == r and bool(np.array_equal(a[3 * mr + 4 * ms:3 * mr + 4 * ms + n_out],
                                                               np.arange(n_out, dtype=np.int32)))
        self.seqs = list(seqs)

    @property
    def max_visible_launch(self) -> int:
        return self.max_context if self.graph_static else self.max_visible

    def upload(self) -> None:
        self.d_int.copy_(self.h_int, non_blocking=True)
        self.d_samp.copy_(self.h_samp, non_blocking=True)

    def h2d_bytes(self) -> int:
        return self.h_int.numel() * 4 + self.h_samp.numel()
