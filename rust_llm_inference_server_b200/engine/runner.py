"""The step function: one batch of (request, its next tokens), portions of prompts beside single
decoded tokens, run from the cache; logits at the wanted places.

Role of `Engine::step` + `Llama::forward_batch` + `PagedBatch::new`
(crates/engine/src/engine.rs:617-726, crates/model/src/llama.rs:218-286,
crates/model/src/paged.rs:256-296).  Differences by design: logits only where they are asked for
(the reference runs its LM head on every sequence's last row, llama.rs:279-285), and one upload
of all index arrays per step.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..ops import profile


class StepError(ValueError):
    """A batch the step function refuses before anything is launched."""


class _CaptureAbort(Exception):
    """A scratch buffer would have to grow while a graph is being recorded."""


@dataclass
class StepEntry:
    seq_id: int
    tokens: list                    # the request's next tokens (at least one)
    start_pos: int                  # how many of its tokens are already in the cache
    want: list = field(default_factory=list)   # places among `tokens` whose logits are wanted


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepContext:
    """Index arrays of one step on the device, and the step's scratch buffers."""

    def __init__(self, runner, n_tokens: int, n_seqs: int):
        self._runner = runner
        self.n_tokens = n_tokens
        self.n_seqs = n_seqs
        self.token_ids = self.positions = self.seq_of_token = None
        self.slots: list = []
        self.block_tables: list = []
        self.ctx_lens = self.cu_seqlens = self.state_slots = self.logit_rows = None
        # host copies, one entry per request of the batch
        self.q_lens: list = []          # tokens of the request in this step
        self.starts: list = []          # its tokens already in the cache (0: the request starts here)
        self.q_starts: list = []        # row of its first token among the step's tokens
        self.state_slot_ids: list = []  # its fixed-size state slot
        self.max_q_len = 0
        self.max_ctx_len = 0
        self.all_decode = False
        # single decoded tokens and the rest, for the kernels that treat them differently
        self.n_decode = 0
        self.dec_rows = self.dec_seqs = None      # int32 [n_decode]: token row, batch entry
        self.max_decode_ctx = 0
        self.n_prefill_tokens = 0
        self.prefill_rows = None                  # int32: rows of the tokens of longer entries
        self.n_prefill_tiles = 0
        self.prefill_tiles = None                 # int32 [tiles, 2]: (batch entry, first token of the tile)
        self.n_wanted = 0                         # rows whose logits are asked for
        self.wants_every_row = False              # ... and they are all the step's rows, in order
        self._views = None
        self._token_region = None

    def buffer(self, name: str, shape, dtype) -> torch.Tensor:
        return self._runner.workspace(name, shape, dtype)

    def take_tokens(self, ids: torch.Tensor) -> None:
        """Replaces the step's token ids by `ids` (int32 on the device, one per token), in stream
        order: after the upload of the step's arrays, before its kernels."""
        self._token_region().copy_(ids)

    def materialize(self) -> None:
        """Makes the device arrays of the step (see `ModelRunner.prepare`); idempotent."""
        if self._views is not None:
            self._views()
            self._views = None


class ModelRunner:
    GRAPH_AFTER_STEPS = 2       # eager steps of a decode shape before its graph is captured

    def __init__(self, model, cache_manager, storage, max_seq_len: int):
        self.model = model
        self.cache = cache_manager
        self.storage = storage
        self.device = model.device
        self.max_seq_len = int(max_seq_len)
        self.groups = storage.groups
        self.max_blocks = max(1, max((self.max_seq_len + g.page_size - 1) // g.page_size for g in self.groups)) \
            if self.groups else 1
        self._caches = [storage.layer_cache(c) for c in range(len(model.cache_slot_specs))]
        # tokens of a portion that one CTA of the mixers' prompt kernels takes (None: no tile list)
        self.prefill_tile = model.prefill_tile
        self._states = storage.states
        self._ws: dict[str, torch.Tensor] = {}
        self._meta_host = None
        self._meta_dev = None
        # CUDA graphs of decode-only steps, by (batch, wanted rows, split plan); dropped whenever
        # a buffer they point into is replaced by a larger one
        self.use_graphs = True
        self._graphs: dict = {}
        self._graph_seen: dict = {}     # key -> times seen before its capture
        self._graph_pool = None
        self._upload_done = None
        self._graph_launches = 0
        self._capturing = False

    # ---- scratch memory that keeps its address while it is large enough ----

    def workspace(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._ws.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if self._capturing:
                # (graphs cannot be dropped while one is being recorded; the step runs eagerly instead,
                # which sizes the buffer, and the shape is captured the next time it comes)
                raise _CaptureAbort(name)
            cap = max(n, 2 * buf.numel() if buf is not None and buf.dtype == dtype else n)
            self._drop_graphs()         # captured graphs point at the old buffer
            buf = torch.empty((cap,), dtype=dtype, device=self.device)
            self._ws[name] = buf
        return buf[:n].view(*shape)

    def _drop_graphs(self) -> None:
        self._graphs.clear()
        self._graph_pool = None         # a pool dies with its last graph; the next capture opens a new one

    def _meta(self, n: int):
        if self._meta_host is None or self._meta_host.numel() < n:
            cap = max(n, 1 << 16)
            self._drop_graphs()
            self._meta_host = torch.empty((cap,), dtype=torch.int32, pin_memory=True)
            self._meta_dev = torch.empty((cap,), dtype=torch.int32, device=self.device)
        return self._meta_host, self._meta_dev

    # ---- the step ----

    def prepare(self, entries: list) -> StepContext:
        """Checks the batch and uploads its index arrays (one copy)."""
        if not entries:
            raise StepError("empty batch")
        B = len(entries)
        G = len(self.groups)
        ids, starts, lens = [], [], []
        seen = set()
        want_rows = []
        T = 0
        V = self.model.spec.vocab_size
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.seq_id}: empty sequence in batch")
            if e.seq_id in seen:
                raise StepError(f"request {e.seq_id} appears twice in one batch")
            seen.add(e.seq_id)
            if e.start_pos < 0 or e.start_pos + n > self.max_seq_len:
                raise StepError(f"request {e.seq_id}: sequence of {e.start_pos + n} positions exceeds "
                                f"max_seq_len {self.max_seq_len}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.seq_id}: wanted place {w} is outside its {n} tokens")
                want_rows.append(T + w)
            ids.append(int(e.seq_id))
            starts.append(int(e.start_pos))
            lens.append(n)
            T += n
        W = len(want_rows)
        wants_every_row = W == T and want_rows == list(range(T))
        mb = self.max_blocks
        # layout of the int32 block: see the offsets below; every region starts 16-byte aligned
        o_tok = 0
        o_pos = o_tok + _align4(T)
        o_sot = o_pos + _align4(T)
        o_slots = o_sot + _align4(T)
        Ta = _align4(T)
        o_ctx = o_slots + G * Ta
        o_cu = o_ctx + _align4(B)
        o_ss = o_cu + _align4(B + 1)
        o_rows = o_ss + _align4(B)
        dec_rows, dec_seqs, pf_rows = [], [], []
        k = 0
        for b, n in enumerate(lens):
            if n == 1:
                dec_rows.append(k)
                dec_seqs.append(b)
            else:
                pf_rows.extend(range(k, k + n))
            k += n
        Bd, Tp = len(dec_rows), len(pf_rows)
        pf_tiles = [(b, t0) for b, n in enumerate(lens) if n > 1 for t0 in range(0, n, self.prefill_tile)] \
            if self.prefill_tile else []
        # the tiles with the most keys to read first: the GPU hands out CTAs in this order, and the
        # long ones must not be the last to start
        pf_tiles.sort(key=lambda bt: -(starts[bt[0]] + bt[1]))
        Nt = len(pf_tiles)
        o_dr = o_rows + _align4(max(W, 1))
        o_ds = o_dr + _align4(max(Bd, 1))
        o_pr = o_ds + _align4(max(Bd, 1))
        o_pt = o_pr + _align4(max(Tp if Bd else 0, 1))
        o_bt = o_pt + _align4(max(2 * Nt, 1))
        total = o_bt + G * B * mb
        host, dev = self._meta(total)
        if self._upload_done is not None:
            self._upload_done.synchronize()   # the last step's upload has left the pinned block
        h = host.numpy()
        tok = h[o_tok:o_tok + T]
        k = 0
        for e in entries:
            n = len(e.tokens)
            tok[k:k + n] = e.tokens
            k += n
        if T and (int(tok.min()) < 0 or int(tok.max()) >= V):
            raise StepError(f"token id outside the vocabulary of {V}")
        try:
            self.cache.pack_step(
                ids, starts, lens, h[o_pos:o_pos + T], h[o_sot:o_sot + T],
                h[o_slots:o_slots + G * Ta].reshape(G, Ta), h[o_bt:o_bt + G * B * mb].reshape(G, B, mb),
                h[o_ctx:o_ctx + B], h[o_cu:o_cu + B + 1], h[o_ss:o_ss + B])
        except RuntimeError as err:
            raise StepError(str(err)) from None
        if W:
            h[o_rows:o_rows + W] = want_rows
        if Nt:
            h[o_pt:o_pt + 2 * Nt] = np.asarray(pf_tiles, dtype=np.int32).reshape(-1)
        if Bd:
            h[o_dr:o_dr + Bd] = dec_rows
            h[o_ds:o_ds + Bd] = dec_seqs
            if Tp:
                h[o_pr:o_pr + Tp] = pf_rows
        dev[:total].copy_(host[:total], non_blocking=True)
        if self._upload_done is None:
            self._upload_done = torch.cuda.Event()
        self._upload_done.record()

        st = StepContext(self, T, B)
        st.n_wanted = W
        st.wants_every_row = wants_every_row
        st.q_lens = lens
        st.starts = starts
        st.state_slot_ids = h[o_ss:o_ss + B].tolist()
        st.q_starts = h[o_cu:o_cu + B].tolist()
        st.seq_ids = ids
        st.max_q_len = max(lens)
        st.max_ctx_len = max(s + n for s, n in zip(starts, lens))
        st.all_decode = st.max_q_len == 1
        st.h2d_bytes = total * 4
        st.n_decode = Bd
        st.n_prefill_tokens = Tp
        st.n_prefill_tiles = Nt
        if Bd:
            st.max_decode_ctx = max(starts[b] + 1 for b in dec_seqs)

        def views():
            # The step's arrays as views of the uploaded block.  A step replayed from a graph never
            # looks at them (the graph reads the same addresses), so they are made on demand: a
            # dozen tensor views cost more host time than the rest of this function.
            st.token_ids = dev[o_tok:o_tok + T]
            st.positions = dev[o_pos:o_pos + T]
            st.seq_of_token = dev[o_sot:o_sot + T]
            st.slots = [dev[o_slots + g * Ta:o_slots + g * Ta + T] for g in range(G)]
            st.block_tables = [dev[o_bt + g * B * mb:o_bt + (g + 1) * B * mb].view(B, mb) for g in range(G)]
            st.ctx_lens = dev[o_ctx:o_ctx + B]
            st.cu_seqlens = dev[o_cu:o_cu + B + 1]
            st.state_slots = dev[o_ss:o_ss + B]
            st.logit_rows = dev[o_rows:o_rows + W] if W else None
            if Nt:
                st.prefill_tiles = dev[o_pt:o_pt + 2 * Nt].view(Nt, 2)
            if Bd:
                st.dec_rows = dev[o_dr:o_dr + Bd]
                st.dec_seqs = dev[o_ds:o_ds + Bd]
                st.prefill_rows = dev[o_pr:o_pr + Tp] if Tp else None

        st._views = views
        st._token_region = lambda: dev[o_tok:o_tok + T]
        return st

    def _forward_eager(self, st: StepContext):
        st.materialize()
        resid, delta = self.model.forward(st, self._caches, self._states)
        if st.logit_rows is None:
            return None
        return self.model.logits(resid, delta, st, st.logit_rows)

    def _graph_key(self, st: StepContext):
        """Decode-only steps of a model whose parts read nothing from the host run from a captured
        graph: the launch-bound inner loop of generation (about ten kernels a layer)."""
        if not (self.use_graphs and st.all_decode and self.model.graph_safe) or profile.enabled:
            return None
        W = st.n_wanted
        # the parts say what else of the step reaches a launch configuration (the number of pieces
        # decode attention cuts the longest context into)
        return (st.n_seqs, W, self.model.launch_variant(st))

    def forward(self, st: StepContext):
        """Launches the model on a prepared step; float32 logits [wanted, vocab] or None.  The
        logits of a step replayed from a graph live in that graph's output buffer until the next
        step with the same shape."""
        key = self._graph_key(st)
        if key is None:
            return self._forward_eager(st)
        entry = self._graphs.get(key)
        if entry is None:
            # The first steps of a shape run eagerly (which also sizes every scratch buffer for it);
            # a capture costs tens of milliseconds, so shapes that only pass by (a batch that is
            # shrinking as requests finish) never pay it.
            seen = self._graph_seen.get(key, 0)
            if seen < self.GRAPH_AFTER_STEPS:
                self._graph_seen[key] = seen + 1
                return self._forward_eager(st)
            entry = self._capture(st)
            if entry is None:                   # not this time: the step runs as it is
                return self._forward_eager(st)
            self._graphs[key] = entry
        graph, logits, n = entry
        graph.replay()
        self._graph_launches += n
        return logits

    def _capture(self, st: StepContext):
        """Records the step into a CUDA graph: (graph, its logits buffer, launches it holds), or None
        when the recording had to be given up.  While a stream records, freeing device memory or
        another graph is not allowed, and Python's collector may do just that when it meets a dead
        engine: it is held off for the duration."""
        before = ops.launch_count
        counts = dict(ops.launches_by_kernel)
        graph = torch.cuda.CUDAGraph()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        torch.cuda.synchronize()
        collecting = gc.isenabled()
        gc.disable()
        self._capturing = True
        try:
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = self._forward_eager(st)
        except _CaptureAbort:
            return None
        finally:
            self._capturing = False
            if collecting:
                gc.enable()
            n = ops.launch_count - before
            ops.launch_count = before           # recording launches nothing
            ops.launches_by_kernel.clear()
            ops.launches_by_kernel.update(counts)
        return graph, logits, n

    def step(self, entries: list):
        return self.forward(self.prepare(entries))

    def sample(self, logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor | None = None):
        """One token id per row of logits on the device (greedy or Gumbel-max; see ops.sample_rows)."""
        return ops.sample_rows(logits, params, out)

    @property
    def launches(self) -> int:
        """Launches of this package's kernels so far (a graph replay counts the launches it holds)."""
        return ops.launch_count + self._graph_launches
