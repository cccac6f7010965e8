"""Batched data feeding for SNetwork.fit-style training loops (lib/nets/snet.dart:71-85).

The reference's fit() walks host lists sample by sample and, on the CUDA path, stages every operand through
pageable buffers with blocking copies (lib/cuda/cudacaller.dart:32-58).  Here the training set stays in host
memory (numpy), and a feeder moves one batch at a time:

  host rows --threaded gather (fml_stage_rows)--> page-locked staging[b] --copy lane 0, async--> device batch[b]      (b = step % 2)

Two staging buffers and two device buffers per stream of data: while the kernels of batch s execute on the
context's stream, batch s+1 is copied host->device on the lane and batch s+2 is gathered into staging memory by
background host threads (fml_stage_rows_async), so the calling thread only enqueues.  Ordering is carried by the
library's numbered events: the copy lane waits for "kernels of the step that last used set b are done" before it
overwrites device set b, the main stream waits for "upload of set b is done" before the step's first kernel.
A staging buffer is refilled only after the copy that read it has finished (fml_event_sync on that upload's event).
"""
from __future__ import annotations

from typing import Iterator, Optional, Sequence, Tuple

import numpy as np

from ._lib import Context, DeviceArray

# first of the four event slots of the library's pool (0..63) a feeder owns by default: "uploaded" +0 / +1 per
# buffer set, then "consumed" +2 / +3
_EV_UPLOADED = 46
_LANE = 0


class BatchFeeder:
    """Iterates over (inputs, targets) batches as device arrays, prefetching the next batch.

    `arrays` are host arrays that share their first dimension (the sample axis); float arrays are fed as
    float32, integer arrays (labels, token ids) as int32.  `order` is an optional permutation of the sample
    indices (a seeded shuffle is the caller's business: the feeder itself is deterministic).  The last batch
    may be smaller; `drop_last` skips it.

    The device arrays handed out by one iteration are overwritten two iterations later, so a consumer must not
    keep them across steps (the training loop does not: the tape of a step is dropped by backward())."""

    def __init__(self, ctx: Context, arrays: Sequence[np.ndarray], batch_size: int, drop_last: bool = False,
                 event_slots: int = _EV_UPLOADED):
        """`event_slots`: first of four consecutive slots of the context's event pool this feeder owns; two feeders
        that are iterated at the same time on one context (training and validation, say) need different ones."""
        assert len(arrays) > 0 and batch_size > 0
        assert 0 <= event_slots <= 60
        self._ev_uploaded, self._ev_consumed = event_slots, event_slots + 2
        self.ctx, self.batch_size, self.drop_last = ctx, int(batch_size), drop_last
        self.n = int(arrays[0].shape[0])
        self.host = []
        self.kinds = []   # source element type for the staging gather: 0 f32, 1 f64, 2 i32, 3 i64
        for a in arrays:
            a = np.asarray(a)
            assert a.shape[0] == self.n, "all arrays share the sample axis"
            if a.dtype not in (np.float32, np.float64, np.int32, np.int64):
                a = a.astype(np.int64 if np.issubdtype(a.dtype, np.integer) else np.float32)
            self.host.append(np.ascontiguousarray(a))
            self.kinds.append({np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 2,
                               np.dtype(np.int64): 3}[self.host[-1].dtype])
        self.dtypes = [np.int32 if k >= 2 else np.float32 for k in self.kinds]
        self.row_shapes = [tuple(a.shape[1:]) for a in self.host]
        self.row_elems = [int(np.prod(s)) if s else 1 for s in self.row_shapes]
        B = self.batch_size
        # [set][array]
        self.staging = [[ctx.pinned((B,) + s, dt) for s, dt in zip(self.row_shapes, self.dtypes)] for _ in range(2)]
        self.device = [[ctx.empty(*((B,) + s), dtype=dt) for s, dt in zip(self.row_shapes, self.dtypes)] for _ in range(2)]
        self.h2d_bytes = 0          # bytes copied host->device since construction
        self._used = [False, False]  # set b has been consumed by a step at least once
        self._index_alive = [None, None]

    def __len__(self):
        full, rem = divmod(self.n, self.batch_size)
        return full + (1 if rem and not self.drop_last else 0)

    # -- staging and upload ---------------------------------------------------------------------------------------
    def _stage(self, b: int, idx: np.ndarray, background: bool):
        """Gather + narrow the rows `idx` into staging set b on the library's host threads; with `background` the call
        returns at once and fml_stage_wait completes it."""
        c, L = self.ctx, self.ctx.lib
        rows = len(idx)
        contiguous = rows > 0 and int(idx[-1]) - int(idx[0]) == rows - 1 and (rows == 1 or bool(np.all(np.diff(idx) == 1)))
        index = None if contiguous else np.ascontiguousarray(idx, dtype=np.int64)
        self._index_alive[b] = index      # read by the background threads until fml_stage_wait
        fn = L.fml_stage_rows_async if background else L.fml_stage_rows
        for a, st, kind, per_row in zip(self.host, self.staging[b], self.kinds, self.row_elems):
            c.check(fn(c.h, st.ctypes.data, a.ctypes.data, kind, per_row,
                       None if index is None else index.ctypes.data, int(idx[0]) if rows else 0, rows, 0))

    def _upload(self, b: int, rows: int):
        c, L = self.ctx, self.ctx.lib
        if self._used[b]:
            c.check(L.fml_wait_event(c.h, _LANE, self._ev_consumed + b))   # kernels that read device set b are done
        for st, dev, per_row in zip(self.staging[b], self.device[b], self.row_elems):
            n = rows * per_row
            # one call per array; 4-byte elements either way, so the float entry point moves int32 ids as well
            c.check(L.fml_lane_h2d(c.h, _LANE, dev.ptr, st.ctypes.data, n))
            self.h2d_bytes += 4 * n
        c.check(L.fml_event_record_on(c.h, self._ev_uploaded + b, _LANE))

    def batches(self, order: Optional[np.ndarray] = None) -> Iterator[Tuple[DeviceArray, ...]]:
        """Three stages run concurrently once the pipeline is full: the kernels of batch s (context's stream), the
        upload of batch s+1 (copy lane) and the gather of batch s+2 into staging memory (host threads)."""
        c, L = self.ctx, self.ctx.lib
        order = np.arange(self.n) if order is None else np.asarray(order)
        B = self.batch_size
        cuts = [(s, min(s + B, len(order))) for s in range(0, len(order), B)]
        if self.drop_last and cuts and cuts[-1][1] - cuts[-1][0] < B:
            cuts.pop()
        if not cuts:
            return
        rows_of = lambda s: order[cuts[s][0]:cuts[s][1]]
        # the staging buffers may still be the source of a copy issued by an earlier epoch
        c.check(L.fml_lane_sync(c.h, _LANE))
        try:
            self._stage(0, rows_of(0), background=False)
            self._upload(0, len(rows_of(0)))
            if len(cuts) > 1:
                self._stage(1, rows_of(1), background=True)
            for s, (lo, hi) in enumerate(cuts):
                b = s % 2
                if s + 1 < len(cuts):
                    c.check(L.fml_stage_wait(c.h))                     # batch s+1 is in staging set 1-b
                    self._upload(1 - b, cuts[s + 1][1] - cuts[s + 1][0])
                    if s + 2 < len(cuts):
                        # staging set b is the source of the upload of batch s, enqueued one step ago: wait for that
                        # copy alone (the upload of s+1 keeps running), then gather batch s+2 behind the host's back
                        c.check(L.fml_event_sync(c.h, self._ev_uploaded + b))
                        self._stage(b, rows_of(s + 2), background=True)
                c.check(L.fml_wait_event(c.h, -1, self._ev_uploaded + b))
                rows = hi - lo
                yield tuple(dev if rows == B else dev.view(0, (rows,) + shp)
                            for dev, shp in zip(self.device[b], self.row_shapes))
                # everything the consumer enqueued on the main stream for this batch precedes this record
                c.check(L.fml_event_record_on(c.h, self._ev_consumed + b, -1))
                self._used[b] = True
        finally:
            L.fml_stage_wait(c.h)      # also when the consumer stops early: no thread may outlive the arrays it reads
            # A consumer that leaves early (break, exception) never reaches the record behind its last yield: record both
            # device sets as consumed after everything now queued on the main stream, so that the next epoch's uploads
            # wait for the abandoned step's kernels instead of the stale event of an older step.
            for b in range(2):
                L.fml_event_record_on(c.h, self._ev_consumed + b, -1)
