"""The kernel set of the engine: thin Python wrappers that hand tensors' addresses, sizes
and the current stream to the compiled sm_100a kernels.

This is the only kernel set the product has. It needs a CUDA device of compute capability
10.x and the compiled library, and raises when either is missing.
"""

from __future__ import annotations

import contextlib
import functools

import torch

from . import library
from .library import KernelError, check

_F32, _BF16 = 0, 1


def _flag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dtype}")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _timed(kind: str):
    """Marks a kernel-set method as one class of the step's time. While `begin_timing()` is
    in force the outermost such call is bracketed by CUDA events and booked under `kind`;
    otherwise the method runs as it is."""
    def wrap(method):
        @functools.wraps(method)
        def run(self, *args, **kwargs):
            if self._timing is None or self._timing_depth:
                return method(self, *args, **kwargs)
            label = self._timing_label or kind
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._timing_depth += 1
            start.record()
            try:
                return method(self, *args, **kwargs)
            finally:
                stop.record()
                self._timing_depth -= 1
                self._timing.append((label, start, stop))
        return run
    return wrap


class CudaOps:
    def __init__(self, device="cuda", decode_splits: int | None = None, gemm: str = "auto",
                 dependent_launch: bool = False):
        """`gemm` picks the bfloat16 product on many tokens: "tcgen05" (this package's
        TMA + tensor-memory kernel wherever it takes the shape), "library" (cuBLAS through
        torch.mm, where the reference calls F.linear), "auto" (the default: the gated gate/up
        product with its SiLU epilogue on the persistent tcgen05 kernel, where fusing beats
        library product plus gate kernel, and the plain products on the library, which is
        still ahead there) or "simt" (the CUDA-core kernel). Few tokens always take the weight-streaming
        kernels. The float32 engine always runs the CUDA-core kernel: a library product
        would need its reduced-precision mode switched off process-wide to be a true 32-bit
        product."""
        if gemm not in ("library", "simt", "tcgen05", "auto"):
            raise KernelError(f"unknown gemm choice {gemm!r}")
        self.gemm = gemm
        self.skinny = True     # few-token products go to the weight-streaming kernels
        # ... up to this many weight elements: a larger matrix (the LM head) is bound by HBM
        # alone, and there the library's kernel streams faster (measured on B200 with 8
        # tokens, weights cold: 151936 x 896 in 52 us against 76 us, 5.3 against 3.6 TB/s)
        self.skinny_max_elements = 96 * 1024 * 1024
        # ... and from this many on, weights come by TMA (gemm_skinny.cu: skinny_fed_kernel);
        # only those launches have a wait that can give up and so an error word to look at
        self.fed_min_elements = 12 * 1024 * 1024
        # The gated product of a prompt step runs on pairs of SMs (gemm_pair.cu) from this K
        # on; below it the one-CTA persistent kernel is level or ahead (measured on B200 at
        # 2048 tokens: K 896, 34 us one CTA against 35 us pairs; K 1536, 91 against 86; at 4096
        # tokens, K 3584 and 2 x 18944 rows, 1515 against 1028)
        self.pair_min_k = 1024
        # The gated few-token product asks L2 for the down-proj's matrix while it finishes, up
        # to this many bytes (a matrix that L2 cannot hold beside everything else gains nothing)
        self.look_ahead_max_bytes = 32 * 1024 * 1024
        # ... and from this many tokens on (measured on B200 inside the captured decode step,
        # 0.5B sizes: 16 sequences 0.950 -> 0.907 ms; 8 sequences 0.598 -> 0.605, one sequence
        # 0.566 -> 0.578: with few tokens the kernel is too short for the lines to arrive)
        self.look_ahead_min_tokens = 9
        # ... and beyond this many weight elements the library's product followed by the gate
        # kernel is ahead of both (measured on B200 at 2048 tokens, replayed from a graph:
        # 2 x 4864 x 896, 35 us fused against 43; 2 x 8960 x 1536, 87 against 101;
        # 2 x 18944 x 3584, 503 against 424: there the library's 1.5 PFLOP/s outweigh the
        # gate kernel's extra pass)
        self.gated_max_elements = 64 * 1024 * 1024
        # ... and so it is for small portions, below this many multiply-adds (replayed from a
        # graph: 512 tokens at 0.5B widths 17.5 us fused against 14.9; 1024 tokens 23.5 against
        # 25.2; 256 tokens at 1.5B widths 16.2 against 16.5; 512 tokens 25.4 against 28.5)
        self.gated_min_products = 8 * 10 ** 9
        # "auto": the tensor-memory (tcgen05) kernel for prompt portions of head sizes 64 and
        # 128, the mma.sync kernels for everything else; "mma": the mma.sync kernels only
        self.attention = "auto"
        # the mixed-head attention: "auto" (tensor cores where they take the sizes) or "simt"
        self.mixed_head = "auto"
        # the grouped products of routed experts: mma.sync where the sizes allow (bfloat16,
        # widths in multiples of 8); False leaves them to the CUDA-core kernel
        self.expert_tensor_cores = True
        # ... and from this many (token, choice) pairs on, the library's grouped product
        # (measured on B200, 8192 pairs over 16 experts of 1216 x 896: 850 and 640 TFLOP/s
        # against 190 from mma.sync, whose rate is what bounds this package's kernel)
        self.expert_library = True
        # the per-head products of latent attention from this many tokens on (measured on B200,
        # 2048 tokens, 14 heads of 64 x 128: 29 and 35 us on the CUDA cores per call)
        self.head_product_library = True
        self.head_product_library_min_tokens = 256
        self.expert_library_min_pairs = 1024
        self._grouped_mm = getattr(torch, "_grouped_mm", None) or getattr(
            torch.nn.functional, "grouped_mm", None)
        self.mixed_head_blocks_per_sm = 4
        self.mixed_head_max_splits = 32
        self.prompt_cluster: int | None = None  # override of the CTAs per row tile (1, 2, 4)
        # decode-like batches: the key ranges of a (sequence, KV head) as one cluster of up to
        # 8 blocks, merged through distributed shared memory, while fewer than 32 ranges are
        # wanted; beyond that (very long contexts in a small batch) the ranges go through
        # global memory as before
        self.decode_clusters = True
        self.prompt_splits: int | None = None   # override of the key split of prompt portions
        # Normalising inside the consuming product saves a launch but makes every block
        # redo the row statistics; measured on B200 the separate norm kernel is faster for
        # the Qwen2 shapes, so the fusion is off unless asked for.
        self.fuse_norm = False
        # The product that adds into the stream also leaves the stream times the next norm's
        # weight and the rows' sums of squares; the product after that norm multiplies its
        # result rows by 1/rms. The norm's own launch disappears.
        self.fuse_next_norm = True
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the engine's kernels are CUDA only and there is "
                              "no CPU path")
        self.device = torch.device(device)
        major, _minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}x")
        self.lib = library.load()
        # the checked variant of the library (MERCURY_B200_BOUNDS_CHECK=1): indices are
        # compared with their limits inside the kernels; see csrc/common.cuh
        self.checked = bool(self.lib.mb_check_enabled())
        self.lib.mb_gemm_skinny_set_fed_min(self.fed_min_elements)
        # let each kernel be scheduled while its predecessor drains (see csrc/common.cuh)
        self.dependent_launch = bool(dependent_launch)     # True: on every launch, not only in graphs
        self.lib.mb_set_dependent_launch(int(dependent_launch))
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.decode_splits = decode_splits
        # Key ranges per (sequence, KV head) of a captured decode step, whose grid is fixed at
        # capture. Measured on B200 at 2048-token contexts: about `graph_blocks_per_sm_small`
        # blocks per SM while the batch brings at most `graph_small_rows` (sequence, KV head)
        # pairs, at most `graph_max_ranges_small` ranges each (a range then still holds three
        # or more 64-key tiles); about `graph_blocks_per_sm_large` per SM beyond that.
        self.graph_small_rows = 16
        self.decode_long_ranges: bool | None = None   # override of the choice of `_long_ranges`
        self.graph_max_ranges_small = 12
        self.graph_blocks_per_sm_small = 1
        self.graph_blocks_per_sm_large = 2
        self._scratch: torch.Tensor | None = None
        # scratch and counters that a larger request replaced: graphs captured earlier still
        # write to them, so they are never given back to the allocator
        self._retired: list[torch.Tensor] = []
        self._counters: torch.Tensor | None = None   # zeroed tickets of the in-kernel split merge
        self._tc_error: torch.Tensor | None = None   # error word of the tcgen05 kernels
        self._tc_pending = False
        self._argmax_scratch: torch.Tensor | None = None
        self._router_logits: torch.Tensor | None = None
        self._scan_scratch: torch.Tensor | None = None
        # the state-space scan of a long portion in runs walked side by side (from 512 tokens on:
        # below that the sequential walk is as fast and is one launch)
        self.scan_runs = True
        self.scan_runs_min_tokens = 512
        self._float_biases: dict = {}
        self._timing: list | None = None      # (kind, start event, stop event) while timing
        self._timing_depth = 0
        self._event_overhead_ms: float | None = None
        self._timing_label: str | None = None  # overrides the class of the calls inside `_as`
        self._pinned_stream: int | None = None
        self.launches = 0
        self.library_calls = 0
        # Which launch (by count) last wrote a float32 residual stream. A residual product
        # reads the stream before it waits for the kernel in front (see mb_gemm_skinny) unless
        # that kernel is this writer. Only this library's kernels let their successor start
        # early, and each of them that writes a stream is noted here.
        self._last_stream_write = -1
        # split-K partial sums stay float32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # ------------------------------------------------------------------ helpers

    def _stream(self) -> int:
        if self._pinned_stream is not None:
            return self._pinned_stream
        return torch.cuda.current_stream(self.device).cuda_stream

    def set_dependent_launch(self, enabled: bool) -> None:
        """Launch the kernels that follow with (or without) the programmatic-serialization
        attribute; see csrc/common.cuh."""
        self.lib.mb_set_dependent_launch(int(bool(enabled) or self.dependent_launch))

    def pin_stream(self) -> None:
        """Look the current stream up once for the many launches of a step."""
        self._pinned_stream = torch.cuda.current_stream(self.device).cuda_stream

    def unpin_stream(self) -> None:
        self._pinned_stream = None

    @contextlib.contextmanager
    def _as(self, label: str):
        """Calls made inside are booked under `label` instead of their own class."""
        before, self._timing_label = self._timing_label, label
        try:
            yield
        finally:
            self._timing_label = before

    def begin_timing(self) -> None:
        """From now on bracket every kernel-set call with CUDA events (eager steps only: a
        replayed graph makes no calls)."""
        self._timing = []

    def end_timing(self) -> dict[str, float]:
        """Milliseconds per class of call since `begin_timing()`; waits for the device. What
        a pair of events measures with nothing between them (a few microseconds) is taken
        off every call."""
        events, self._timing = self._timing or [], None
        if events and self._event_overhead_ms is None:
            empty = []
            for _ in range(20):
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                stop.record()
                empty.append((start, stop))
            torch.cuda.synchronize(self.device)
            gaps = sorted(a.elapsed_time(b) for a, b in empty)
            self._event_overhead_ms = gaps[len(gaps) // 2]
        torch.cuda.synchronize(self.device)
        out: dict[str, float] = {}
        for kind, start, stop in events:
            out[kind] = out.get(kind, 0.0) + max(0.0, start.elapsed_time(stop) - self._event_overhead_ms)
        return out

    def _scratch_for(self, floats: int) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < floats:
            if self._scratch is not None:
                # a captured graph may hold the old buffer's address: keep it allocated
                self._retired.append(self._scratch)
            self._scratch = torch.empty(max(floats, 1 << 20), dtype=torch.float32,
                                        device=self.device)
        return self._scratch

    def _scan_scratch_for(self, floats: int) -> torch.Tensor:
        if self._scan_scratch is None or self._scan_scratch.numel() < floats:
            if self._scan_scratch is not None:
                self._retired.append(self._scan_scratch)
            self._scan_scratch = torch.empty(max(floats, 1 << 20), dtype=torch.float32,
                                             device=self.device)
        return self._scan_scratch

    def _counters_for(self, count: int) -> torch.Tensor:
        """Zeroed tickets of the in-kernel split merge (the last block resets its own)."""
        if self._counters is None or self._counters.numel() < count:
            if self._counters is not None:
                self._retired.append(self._counters)
            self._counters = torch.zeros(max(count, 4096), dtype=torch.int32, device=self.device)
        return self._counters

    @staticmethod
    def _rows(t: torch.Tensor) -> torch.Tensor:
        if not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")
        return t

    # ------------------------------------------------------------------ kernels

    @_timed("embedding")
    def embed(self, token_ids, table, out, positions=None, position_table=None, scale=1.0):
        """out = table[token_ids] (+ position_table[positions]) in the float32 stream; with
        `scale` (and no positions) every row is multiplied by it."""
        self._rows(out)
        if scale != 1.0:
            if position_table is not None:
                raise KernelError("embed: a scale together with learned positions is not built")
            check(self.lib.mb_embed_scaled(_ptr(token_ids), _ptr(table), _flag(table.dtype),
                                           float(scale), _ptr(out), out.shape[0], out.shape[1],
                                           table.shape[0], self._stream()), "embed")
        elif position_table is None:
            check(self.lib.mb_embed(_ptr(token_ids), _ptr(table), _flag(table.dtype), _ptr(out),
                                    out.shape[0], out.shape[1], table.shape[0], self._stream()),
                  "embed")
        else:
            check(self.lib.mb_embed_positions(
                _ptr(token_ids), _ptr(table), _flag(table.dtype), _ptr(positions),
                _ptr(position_table), _flag(position_table.dtype), position_table.shape[0],
                _ptr(out), out.shape[0], out.shape[1], table.shape[0], self._stream()), "embed")
        self.launches += 1
        self._note_stream_write()

    @_timed("norm")
    def rmsnorm_add(self, h, delta, weight, eps, next_weight, next_eps, out, delta2=None,
                    scale=1.0, scale2=1.0, tail=None):
        """h += rmsnorm(delta) * weight (a norm behind a sublayer); with `next_weight` also
        out = rmsnorm(h) * next_weight of the new stream, in the same kernel. With `delta2` or a
        `scale` the norm is taken of scale * delta + scale2 * delta2 (two sublayers that ran
        side by side)."""
        self._rows(h), self._rows(delta)
        if delta2 is not None or scale != 1.0 or tail is not None:
            if next_weight is not None:
                raise KernelError("rmsnorm_add: two deltas together with the next norm are not built")
            if delta2 is not None:
                self._rows(delta2)
                if delta2.dtype != delta.dtype or delta2.shape != delta.shape:
                    raise KernelError("rmsnorm_add: the two deltas differ in type or shape")
            # `tail` = (ring, batch): the stream's rows as the sublayer found them, a sequence's
            # last ones, go into the ring of the convolution in front of the sublayer
            ring, batch = tail if tail is not None else (None, None)
            check(self.lib.mb_rmsnorm_add_pair(
                _ptr(h), _ptr(delta), _ptr(delta2), _flag(delta.dtype), float(scale), float(scale2),
                _ptr(weight), _flag(weight.dtype), float(eps), h.shape[0], h.shape[1],
                _ptr(ring), ring.stride(0) if ring is not None else 0,
                ring.shape[1] if ring is not None else 0,
                _ptr(batch.positions) if ring is not None else None,
                _ptr(batch.seq_of_token) if ring is not None else None,
                _ptr(batch.kv_len) if ring is not None else None,
                _ptr(batch.slots) if ring is not None else None,
                self._stream()), "rmsnorm_add (pair)")
            self.launches += 1
            self._note_stream_write()
            return
        check(self.lib.mb_rmsnorm_add(
            _ptr(h), _ptr(delta), _flag(delta.dtype), _ptr(weight), _flag(weight.dtype), float(eps),
            _ptr(next_weight), _flag(next_weight.dtype) if next_weight is not None else 0,
            float(next_eps), _ptr(out), _flag(out.dtype) if out is not None else 0,
            h.shape[0], h.shape[1], self._stream()), "rmsnorm_add")
        self.launches += 1
        self._note_stream_write()

    @_timed("embedding")
    def embed_bigram(self, token_ids, table, pairs, buckets, mul_prev, mul_cur, state, batch, out):
        """out = table[token] + pairs[(previous * mul_prev + token * mul_cur) mod buckets] (row
        `buckets` for a sequence's first token) in the float32 stream; `state` [slots, 1] int32
        holds every live sequence's last token and is brought up to date."""
        self._rows(out)
        if state.dtype != torch.int32 or pairs.shape[0] != buckets + 1:
            raise KernelError("embed_bigram: the state is int32 and the pair table has buckets + 1 rows")
        check(self.lib.mb_embed_bigram(
            _ptr(token_ids), _ptr(table), _flag(table.dtype), _ptr(pairs), _flag(pairs.dtype),
            int(buckets), int(mul_prev), int(mul_cur), _ptr(batch.positions), _ptr(batch.seq_of_token),
            _ptr(batch.q_start), _ptr(batch.slots), _ptr(state), state.stride(0), _ptr(out),
            out.shape[0], out.shape[1], table.shape[0], self._stream()), "embed_bigram")
        self.launches += 1
        self._note_stream_write()

    @_timed("norm")
    def rmsnorm_join_add(self, h, x, y, wx, wy, a, b, weight, eps, next_weight, next_eps, out):
        """h += rmsnorm(a n(x) + b n(y)) * weight with n(x) = rmsnorm(x) * wx (x itself where wx is
        None), likewise n(y): two sublayer outputs that ran side by side, normed each, joined,
        and the norm behind the sublayer, in one pass. With `next_weight` also out = rmsnorm(h) *
        next_weight of the new stream. All weights float32."""
        self._rows(h), self._rows(x), self._rows(y)
        if x.dtype != y.dtype or x.shape != y.shape:
            raise KernelError("rmsnorm_join_add: the two outputs differ in type or shape")
        for w in (wx, wy, weight, next_weight):
            if w is not None and w.dtype != torch.float32:
                raise KernelError("rmsnorm_join_add: the norm weights are float32")
        check(self.lib.mb_rmsnorm_join_add(
            _ptr(h), _ptr(x), _ptr(y), _flag(x.dtype), _ptr(wx), _ptr(wy), float(a), float(b),
            _ptr(weight), float(eps), _ptr(next_weight), float(next_eps), _ptr(out),
            _flag(out.dtype) if out is not None else 0, h.shape[0], h.shape[1], self._stream()),
            "rmsnorm_join_add")
        self.launches += 1
        self._note_stream_write()

    def _note_stream_write(self) -> None:
        self._last_stream_write = self.launches + self.library_calls

    def patch_tokens(self, token_ids, token_from, sampled):
        """token_ids[t] = sampled[token_from[t]] wherever token_from[t] >= 0: ids that the
        step before has sampled on the device and the host has not read yet."""
        check(self.lib.mb_patch_tokens(_ptr(token_ids), _ptr(token_from), _ptr(sampled),
                                       token_ids.shape[0], self._stream()), "patch_tokens")
        self.launches += 1

    @_timed("norm")
    def add_rmsnorm(self, h, delta, weight, eps, out, rows=None):
        count = h.shape[0] if rows is None else rows.shape[0]
        if delta is not None and delta.dtype != out.dtype:
            raise KernelError("add_rmsnorm: delta and out must share the activation dtype")
        check(self.lib.mb_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), _flag(weight.dtype),
                                      _ptr(out), _ptr(rows), count, h.shape[1], float(eps),
                                      _flag(out.dtype), self._stream()), "add_rmsnorm")
        self.launches += 1
        if rows is None:
            self._note_stream_write()

    def _error_word(self) -> torch.Tensor:
        if self._tc_error is None:
            self._tc_error = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._tc_error

    def _check_limits(self, cache, tables=None) -> None:
        """Checked build: tell the kernels that follow how many pages the pool of `cache`
        has and how many rows the rotation tables have."""
        if self.checked and cache is not None:
            rows = tables[0].shape[0] if tables is not None else 0
            check(self.lib.mb_check_set_limits(cache.k.shape[0], rows, self._stream()),
                  "check limits")

    def check_errors(self) -> None:
        """Raise if a bounded wait inside a tcgen05 kernel ran out since the last check
        (reads one word from the device, so it synchronises). In the checked build also
        raise if a kernel met an index beyond its limit."""
        if self.checked:
            import ctypes

            word = (ctypes.c_int * 4)()
            check(self.lib.mb_check_read(word, self._stream()), "check read")
            if word[0]:
                kind = {1: "a page number beyond the pool", 2: "a block-table column beyond the table",
                        3: "a position beyond the rotation tables", 4: "a token id outside the vocabulary",
                        5: "a sequence number beyond the batch"}.get(word[0], f"kind {word[0]}")
                raise KernelError(f"bounds check: {kind}: {word[1]} (limit {word[2]}), "
                                  f"{word[3]} bad indices in all; the accesses were skipped")
        if not self._tc_pending or self._tc_error is None:
            self._tc_pending = False
            return
        self._tc_pending = False
        code = int(self._tc_error.item())
        if code:
            self._tc_error.zero_()
            role = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue or the softmax",
                    4: "the producer's drain or the wait for the output", 5: "the MMA issuer (P)",
                    6: "the meeting of a row's two softmax threads",
                    7: "a weight ring of a few-token product",
                    8: "the key tiles of the decode attention"}.get(code, f"code {code}")
            raise KernelError(f"a kernel gave up waiting in {role}; its output is invalid")

    # -- inputs that may still be an unevaluated norm (parts/norm.py: PendingNorm)

    def can_fuse_norm(self, rows: int, hidden: int, weight) -> bool:
        """Whether a few-token product can normalise its own input for this shape."""
        return (self.fuse_norm and self.skinny and rows <= 16 and hidden % 32 == 0
                and weight.dtype == torch.bfloat16)

    @staticmethod
    def _pending(x):
        return x if hasattr(x, "materialize") else None

    def _skinny_input(self, x):
        """The nine input arguments of the few-token products: (x, h, norm weight, rows, eps)
        and (partial sums of squares, their tiles per row, eps, row length)."""
        pending = self._pending(x)
        if pending is None:
            return _ptr(x), None, None, None, 0.0, None, 0, 0.0, 0
        scaled = getattr(pending, "ss_part", None)
        if scaled is not None:
            return (_ptr(pending.x), None, None, None, 0.0, _ptr(scaled), scaled.shape[1],
                    float(pending.eps), pending.size)
        return (None, _ptr(pending.h), _ptr(pending.weight), _ptr(pending.rows), float(pending.eps),
                None, 0, 0.0, 0)

    @_timed("residual product")
    def linear_residual(self, x, weight, bias, h, ctx, name, then_norm=None):
        """h += x . weight^T (+ bias) in the float32 stream when the few-token kernel takes
        the shape (returns None); otherwise the product lands in the buffer `name` and is
        returned for the next norm to add. `then_norm` names the norm part that follows
        (it has `weight`, `eps`, `size`): the kernel then also leaves that norm's output, up
        to the division by the row's rms, in `ctx.prenormed` (a `PendingScaled`), where the
        norm part picks it up instead of launching."""
        m, k = x.shape
        n = weight.shape[0]
        if (self.skinny and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and (bias is None or bias.dtype == torch.bfloat16) and h.dtype == torch.float32
                and self.lib.mb_gemm_skinny_supports(m, n, k)):
            fuse = (then_norm is not None and self.fuse_next_norm and n % 4 == 0
                    and getattr(then_norm, "size", None) == n
                    and getattr(then_norm, "weight", None) is not None
                    and then_norm.weight.dtype == torch.bfloat16)
            normed = ctx.buffer("normed", m, n) if fuse else None
            sums = ctx.buffer("norm_sums", m, n // 16, dtype="float32") if fuse else None
            stable = self._last_stream_write != self.launches + self.library_calls
            check(self.lib.mb_gemm_skinny(
                *self._skinny_input(x), _ptr(weight), _ptr(bias), _ptr(h), 3, m, n, k,
                _ptr(then_norm.weight) if fuse else None, _ptr(normed), _ptr(sums), int(stable),
                _ptr(self._error_word()), self._stream()), "linear_residual (skinny)")
            self.launches += 1
            self._tc_pending = self._tc_pending or n * k >= self.fed_min_elements
            self._note_stream_write()
            if fuse:
                from ..parts.norm import PendingScaled

                ctx.prenormed = (then_norm, PendingScaled(normed, sums, h, then_norm.weight,
                                                          then_norm.eps, ctx, n))
            return None
        out = ctx.buffer(name, m, n)
        self.linear(x, weight, bias, out)
        return out

    @_timed("product")
    def linear(self, x, weight, bias, out):
        pending = self._pending(x)
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
            raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> "
                              f"{tuple(out.shape)} do not fit")
        self._rows(weight), self._rows(out)
        all_bf16 = (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                    and (bias is None or bias.dtype == torch.bfloat16))
        if (all_bf16 and self.skinny and self.lib.mb_gemm_skinny_supports(m, n, k)
                and (n * k <= self.skinny_max_elements or self.gemm == "simt")):
            check(self.lib.mb_gemm_skinny(*self._skinny_input(x), _ptr(weight), _ptr(bias),
                                          _ptr(out), 0 if out.dtype == torch.bfloat16 else 1, m, n, k,
                                          None, None, None, 0, _ptr(self._error_word()),
                                          self._stream()),
                  "linear (skinny)")
            self.launches += 1
            self._tc_pending = self._tc_pending or n * k >= self.fed_min_elements
            return
        if pending is not None:
            x = pending.materialize()
        self._rows(x)
        if all_bf16 and self.gemm in ("tcgen05", "auto") and self.lib.mb_gemm_tcgen05_supports(m, n, k):
            # Measured inside a 2048-token step on B200 (weights cold in L2) the library is
            # ahead on the plain products (q/k/v 8.5 us, o 7.3 us, down 17 us against 12, 12
            # and 33 us), so "auto" leaves them to it; the gated product is where this
            # package's kernel wins (see linear_swiglu).
            if self.gemm == "tcgen05":
                check(self.lib.mb_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out),
                                               int(out.dtype == torch.float32), m, n, k,
                                               _ptr(self._error_word()), 0, self._stream()),
                      "linear (tcgen05)")
                self.launches += 1
                self._tc_pending = True
                return
        if self.gemm != "simt" and all_bf16:
            return self._library_linear(x, weight, bias, out)
        check(self.lib.mb_gemm_simt(_ptr(x), _flag(x.dtype), _ptr(weight), _flag(weight.dtype),
                                    _ptr(bias), _flag(bias.dtype) if bias is not None else 0,
                                    _ptr(out), _flag(out.dtype), m, n, k, self._stream()),
              "linear")
        self.launches += 1

    def _library_linear(self, x, weight, bias, out):
        """bfloat16 operands, float32 accumulation in cuBLAS; the result is rounded once, to
        bfloat16 or (for logits) kept in float32."""
        if out.dtype == torch.bfloat16:
            if bias is None:
                torch.mm(x, weight.t(), out=out)
            else:
                torch.addmm(bias, x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
            if bias is not None:
                out.add_(self._float_bias(bias))
        self.library_calls += 1

    def _float_bias(self, bias):
        """The float32 copy of a bias, made once per tensor (a product whose result stays
        float32 adds its bias in float32)."""
        key = bias.data_ptr()
        held = self._float_biases.get(key)
        if held is None or held[0] is not bias:
            held = self._float_biases[key] = (bias, bias.float())
        return held[1]

    @_timed("gated product")
    def linear_swiglu(self, x, weight, out, ctx, ahead=None, gate=None):
        """out = silu(x . gate^T) * (x . up^T) for `weight` = [gate rows; up rows]: one kernel
        for few tokens, product then gate otherwise. `ahead`: the matrix that the product
        behind this one will stream; the few-token kernel asks L2 for it once its own weights
        are in (`look_ahead_max_bytes` bounds what is asked for)."""
        m, k = x.shape
        width = out.shape[1]
        # `gate` = (limit, slope): the clamped sigmoid gate in place of SiLU, which only the
        # few-token kernel has fused (None is returned when this call is not for it)
        form = (0, 0.0, 1.0) if gate is None else (2, float(gate[0]), float(gate[1]))
        if (self.skinny and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and self.lib.mb_gemm_skinny_supports(m, width, k)
                and 2 * width * k <= self.skinny_max_elements):
            bytes_ahead = 0
            if (ahead is not None and m >= self.look_ahead_min_tokens and ahead.is_cuda
                    and ahead.is_contiguous()
                    and ahead.numel() * ahead.element_size() <= self.look_ahead_max_bytes):
                bytes_ahead = ahead.numel() * ahead.element_size()
            check(self.lib.mb_gemm_skinny_swiglu(*self._skinny_input(x), _ptr(weight), _ptr(out),
                                                 m, width, k, _ptr(ahead) if bytes_ahead else None,
                                                 bytes_ahead, *form, _ptr(self._error_word()),
                                                 self._stream()),
                  "linear_swiglu (skinny)")
            self.launches += 1
            self._tc_pending = self._tc_pending or 2 * width * k >= self.fed_min_elements
            return True
        if gate is not None:
            return None
        if self._pending(x) is not None:
            x = x.materialize()
        if (self.gemm in ("tcgen05", "auto") and x.dtype == torch.bfloat16
                and weight.dtype == torch.bfloat16 and m >= 256 and width % 8 == 0
                and ((2 * width * k <= self.gated_max_elements
                      and 2 * m * width * k >= self.gated_min_products) or self.gemm == "tcgen05")
                and self.lib.mb_gemm_tcgen05_supports(m, width, k)):
            if k >= self.pair_min_k and self.lib.mb_gemm_pair_supports(m, width, k):
                # pairs of SMs sharing one 256-row MMA: a CTA loads a third less per output
                check(self.lib.mb_gemm_pair(_ptr(x), _ptr(weight), None, _ptr(out), 2, m, width, k,
                                            None, 0, 0.0, 0, None, None, None, None,
                                            _ptr(self._error_word()), self._stream()),
                      "linear_swiglu (tcgen05 pairs)")
            else:
                check(self.lib.mb_gemm_tcgen05_persistent(_ptr(x), _ptr(weight), None, _ptr(out), 2, m,
                                                          width, k, _ptr(self._error_word()),
                                                          self._stream()), "linear_swiglu (tcgen05)")
            self.launches += 1
            self._tc_pending = True
            return
        gate_up = ctx.buffer("gate_up", m, 2 * width)
        self.linear(x, weight, None, gate_up)
        self.swiglu(gate_up, out)

    def linear_gated(self, x, weight, out, ctx, activation, limit=0.0, slope=1.0):
        """out = act(x . gate^T) * (x . up^T) for `weight` = [gate rows; up rows]; "silu" takes
        the fused kernels of `linear_swiglu`, "gelu_tanh" the product followed by the gate
        kernel; "clamped_sigmoid" is g sigmoid(slope g) (u + 1) of g = min(gate, limit) and u =
        clamp(up, -limit, limit), product and gate kernel as well."""
        if activation == "silu":
            return self.linear_swiglu(x, weight, out, ctx)
        if activation not in ("gelu_tanh", "clamped_sigmoid"):
            raise KernelError(f"no gate kernel for the activation {activation!r}")
        if activation == "clamped_sigmoid" and self.linear_swiglu(x, weight, out, ctx,
                                                                  gate=(limit, slope)):
            return           # few tokens: product and gate in one kernel
        if self._pending(x) is not None:
            x = x.materialize()
        m, width = x.shape[0], out.shape[1]
        gate_up = ctx.buffer("gate_up", m, 2 * width)
        with self._as("gated product"):
            self.linear(x, weight, None, gate_up)
        self.gated_act(gate_up, out, 1 if activation == "gelu_tanh" else 2, limit, slope)

    @_timed("gate")
    def gated_act(self, gate_up, out, act: int, limit: float = 0.0, slope: float = 1.0):
        check(self.lib.mb_gated_act(_ptr(gate_up), _ptr(out), out.shape[0], out.shape[1],
                                    _flag(out.dtype), int(act), float(limit), float(slope),
                                    self._stream()), "gated_act")
        self.launches += 1

    # ------------------------------------------------------------------ recurrent mixers

    @_timed("recurrence")
    def mingru_scan(self, pre, state, batch, out):
        """pre [tokens, 3 * width] float32 = [z | u | g] before their activations; the state
        [slots, width] float32 goes from token to token; out [tokens, width]."""
        check(self.lib.mb_mingru_scan(_ptr(pre), _ptr(state), _ptr(batch.q_start), _ptr(batch.slots),
                                      _ptr(out), batch.num_seqs, batch.max_q_len, out.shape[1],
                                      _flag(out.dtype), self._stream()), "mingru_scan")
        self.launches += 1

    @_timed("recurrence")
    def causal_conv(self, pre, offset, width, taps_w, bias, state, batch, u):
        """u = causal convolution per channel of the columns [offset, offset + width) of `pre`
        (float32), the inputs from before the step taken from rows 1.. of the state
        [slots, taps, width]."""
        check(self.lib.mb_causal_conv(_ptr(pre), pre.shape[1], int(offset), _ptr(taps_w), _ptr(bias),
                                      _ptr(state), _ptr(batch.q_start), _ptr(batch.slots),
                                      _ptr(batch.seq_of_token), _ptr(u), u.shape[0], int(width),
                                      taps_w.shape[1], self._stream()), "causal_conv")
        self.launches += 1

    @_timed("recurrence")
    def block_gates(self, u, weight, bias, gates):
        """gates [tokens, kinds * width] = sigmoid of the block-diagonal products of u
        [tokens, width] with weight [kinds, blocks, in, out] + bias [kinds, blocks, out], all
        float32 on the CUDA cores."""
        kinds, blocks = weight.shape[0], weight.shape[1]
        check(self.lib.mb_block_gates(_ptr(u), _ptr(weight), _ptr(bias), _ptr(gates), u.shape[0],
                                      u.shape[1], blocks, kinds, self._stream()), "block_gates")
        self.launches += 1

    @_timed("recurrence")
    def gated_recurrence_scan(self, pre, u, gates, softplus_lam, decay_scale, state, batch, out):
        """S <- a S + sqrt(1 - a^2) i u with a = exp(-decay_scale * r * softplus_lam), out =
        S * gelu_tanh(y); pre = [y | x], gates = [r | i]; the state's rows 1.. (the
        convolution's past inputs) are brought up to the end of the step."""
        check(self.lib.mb_gated_recurrence_scan(
            _ptr(pre), _ptr(u), _ptr(gates), _ptr(softplus_lam), float(decay_scale), _ptr(state),
            _ptr(batch.q_start), _ptr(batch.slots), _ptr(out), batch.num_seqs, batch.max_q_len,
            out.shape[1], state.shape[1], _flag(out.dtype), self._stream()), "gated_recurrence_scan")
        self.launches += 1

    # ------------------------------------------------------------------ stream, layer scale, cap

    @_timed("norm")
    def scaled_add_norm(self, h, delta, scale, weight, eps, center, out, rows=None):
        """h += delta * scale (either may be None); then, if `weight` is given, out = the
        layer norm (`center`) or RMS norm of the new rows times weight. With `rows` only
        those rows are normalised and h is left as it was."""
        self._rows(h)
        count = h.shape[0] if rows is None else rows.shape[0]
        if delta is not None:
            self._rows(delta)
        check(self.lib.mb_scaled_add_norm(
            _ptr(h), _ptr(delta), _flag(delta.dtype) if delta is not None else 0, _ptr(scale),
            _flag(scale.dtype) if scale is not None else 0, _ptr(weight),
            _flag(weight.dtype) if weight is not None else 0, float(eps), int(bool(center)),
            _ptr(out) if weight is not None else None,
            _flag(out.dtype) if (weight is not None and out is not None) else 0, _ptr(rows), count,
            h.shape[1], self._stream()), "scaled_add_norm")
        self.launches += 1
        if rows is None and delta is not None:
            self._note_stream_write()

    @_timed("head")
    def softcap(self, logits, cap):
        """logits <- cap * tanh(logits / cap), in place (float32)."""
        self._rows(logits)
        check(self.lib.mb_softcap(_ptr(logits), logits.numel(), float(cap), self._stream()), "softcap")
        self.launches += 1

    # ------------------------------------------------------------------ state-space, delta rule

    @_timed("recurrence")
    def conv_act(self, pre, offset, conv, bias, tail, batch, out, act):
        """out = act(causal convolution per channel of pre[:, offset : offset + channels] +
        bias), float32; `tail` [slots, (taps - 1) * channels] (a view of the state rows) holds
        the inputs from before the step and is left as it was. act: "silu" or None."""
        channels, taps = conv.shape
        if act not in ("silu", None):
            raise KernelError(f"conv_act: no activation {act!r}")
        check(self.lib.mb_conv_act(
            _ptr(pre), pre.shape[1], int(offset), _ptr(conv), _ptr(bias), _ptr(tail), tail.stride(0),
            _ptr(batch.q_start), _ptr(batch.slots), _ptr(batch.seq_of_token), _ptr(out), out.shape[0],
            channels, taps, 1 if act == "silu" else 0, self._stream()), "conv_act")
        self.launches += 1

    @_timed("recurrence")
    def conv_act_update(self, pre, offset, conv, bias, tail, batch, out, act):
        """`conv_act` and then `conv_tail_update`: one launch for steps of at most 8 tokens a
        sequence (one thread per sequence and channel walks them), two otherwise."""
        channels, taps = conv.shape
        if act not in ("silu", None):
            raise KernelError(f"conv_act: no activation {act!r}")
        check(self.lib.mb_conv_act_update(
            _ptr(pre), pre.shape[1], int(offset), _ptr(conv), _ptr(bias), _ptr(tail), tail.stride(0),
            _ptr(batch.q_start), _ptr(batch.slots), _ptr(batch.seq_of_token), _ptr(out), out.shape[0],
            batch.num_seqs, batch.max_q_len, channels, taps, 1 if act == "silu" else 0,
            self._stream()), "conv_act_update")
        self.launches += 1 if (batch.max_q_len <= 8 or taps <= 1) else 2

    @_timed("recurrence")
    def conv_tail_update(self, pre, offset, channels, taps, tail, batch):
        """Bring the convolution's past inputs up to the end of the step."""
        if taps <= 1:
            return
        check(self.lib.mb_conv_tail_update(
            _ptr(pre), pre.shape[1], int(offset), _ptr(tail), tail.stride(0), _ptr(batch.q_start),
            _ptr(batch.slots), batch.num_seqs, int(channels), int(taps), self._stream()),
            "conv_tail_update")
        self.launches += 1

    @_timed("recurrence")
    def mamba2_scan(self, xbc, pre, dt_offset, dt_bias, neg_rate, skip, layout, cells, batch, y,
                    precise=False):
        """S <- exp(neg_rate dt) S + dt B x^T, y = S^T C + skip x per head, dt = softplus(pre[:,
        dt_offset + head] + dt_bias); xbc = [x | B | C]; `cells` [slots, heads * state * vdim]
        is a view of the state rows; everything float32. `precise`: the matrices are held in
        double while the step runs (the float32 engine; see csrc/state_space.cu)."""
        heads, vdim, n_state, groups = layout
        tokens = xbc.shape[0]
        # long portions are cut into runs that blocks walk side by side (three launches)
        in_runs = self.scan_runs and not precise and batch.max_q_len >= self.scan_runs_min_tokens
        scratch = None
        if in_runs:
            scratch = self._scan_scratch_for(self.lib.mb_mamba2_scratch_floats(
                tokens, batch.num_seqs, batch.max_q_len, heads, vdim, n_state))
        check(self.lib.mb_mamba2_scan(
            _ptr(xbc), _ptr(pre), pre.shape[1], int(dt_offset), _ptr(dt_bias), _ptr(neg_rate),
            _ptr(skip), _ptr(cells), cells.stride(0), _ptr(batch.q_start), _ptr(batch.slots), _ptr(y),
            tokens, batch.num_seqs, batch.max_q_len, heads, vdim, n_state, groups,
            int(bool(precise)), _ptr(scratch), self._stream()), "mamba2_scan")
        self.launches += 3 if in_runs else 1

    @_timed("recurrence")
    def delta_rule_scan(self, qkv, pre, beta_offset, decay_offset, dt_bias, neg_rate, layout,
                        unit_eps, cells, batch, o, precise=False):
        """The gated delta rule per head over qkv = [q | k | v]; beta and the decay are read
        off pre[:, beta_offset + head] and pre[:, decay_offset + head]; `cells` [slots, heads *
        dim * vdim] is a view of the state rows; everything float32 (`precise` as in
        `mamba2_scan`)."""
        heads, key_heads, dim, vdim = layout
        check(self.lib.mb_delta_rule_scan(
            _ptr(qkv), _ptr(pre), pre.shape[1], int(beta_offset), int(decay_offset), _ptr(dt_bias),
            _ptr(neg_rate), float(unit_eps), _ptr(cells), cells.stride(0), _ptr(batch.q_start),
            _ptr(batch.slots), _ptr(o), batch.num_seqs, heads, key_heads, dim, vdim,
            int(bool(precise)), self._stream()), "delta_rule_scan")
        self.launches += 1

    @_timed("recurrence")
    def gated_group_norm(self, y, pre, gate_offset, weight, groups, eps, gate_first, out,
                         gate="silu"):
        """RMS norm of y (float32) in `groups` equal parts times `weight` (read at c modulo its
        length), times silu(pre[:, gate_offset + c]) (`gate` "sigmoid": sigmoid(.)) before
        (`gate_first`) or behind the norm."""
        tokens, width = y.shape
        if gate not in ("silu", "sigmoid"):
            raise KernelError(f"gated_group_norm: no gate {gate!r}")
        flags = int(bool(gate_first)) | (2 if gate == "sigmoid" else 0)
        check(self.lib.mb_gated_group_norm(
            _ptr(y), _ptr(pre), pre.shape[1], int(gate_offset), _ptr(weight), weight.numel(),
            int(groups), width // int(groups), float(eps), flags, _ptr(out),
            _flag(out.dtype), tokens, self._stream()), "gated_group_norm")
        self.launches += 1

    # ------------------------------------------------------------------ generalized delta rule

    @_timed("recurrence")
    def tanh_slice(self, pre, offset, count, out):
        """out = tanh(pre[:, offset : offset + count]), float32."""
        check(self.lib.mb_tanh_slice(_ptr(pre), pre.shape[1], int(offset), int(count), _ptr(out),
                                     pre.shape[0], self._stream()), "tanh_slice")
        self.launches += 1

    @_timed("recurrence")
    def general_delta_scan(self, pre, offsets, decay, decay_scale, layout, unit_eps, cells, batch, o,
                           precise=False):
        """Per head S <- diag(w) S - (a * u)(u^T S) + k v^T, o = S^T r, with w = exp(-decay_scale *
        sigmoid(decay)), a = sigmoid(pre[a]) and u = k / sqrt(sum k^2 + unit_eps); r, k, v and a
        are read off `pre` at `offsets`; `cells` [slots, heads * dim * vdim] holds the matrices;
        everything float32 (`precise` as in `mamba2_scan`)."""
        heads, dim, vdim = layout
        at_r, at_k, at_v, at_a = offsets
        if pre.dtype != torch.float32 or decay.dtype != torch.float32 or o.dtype != torch.float32:
            raise KernelError("general_delta_scan: inputs and read-outs are float32")
        check(self.lib.mb_general_delta_scan(
            _ptr(pre), pre.shape[1], int(at_r), int(at_k), int(at_v), int(at_a), _ptr(decay),
            float(decay_scale), float(unit_eps), _ptr(cells), cells.stride(0), _ptr(batch.q_start),
            _ptr(batch.slots), _ptr(o), batch.num_seqs, heads, dim, vdim, int(bool(precise)),
            self._stream()), "general_delta_scan")
        self.launches += 1

    # ------------------------------------------------------------------ stream convolution

    @_timed("norm")
    def stream_conv(self, h, weight, state, batch, out):
        """out = h + the causal convolution of h per channel (weight [hidden, taps] float32),
        rows from before the step out of the ring `state` [slots, taps - 1, hidden]; without a
        weight out = h. The ring is left as it was."""
        self._rows(h), self._rows(out)
        taps = weight.shape[1] if weight is not None else 1
        if weight is not None and (weight.dtype != torch.float32 or not weight.is_contiguous()):
            raise KernelError("stream_conv: the taps are a contiguous float32 matrix")
        check(self.lib.mb_stream_conv(
            _ptr(h), _ptr(weight), int(taps), _ptr(state), state.stride(0) if state is not None else 0,
            _ptr(batch.positions), _ptr(batch.seq_of_token), _ptr(batch.q_start), _ptr(batch.kv_len),
            _ptr(batch.slots), _ptr(out), _flag(out.dtype), h.shape[0], h.shape[1], self._stream()),
            "stream_conv")
        self.launches += 1

    @_timed("norm")
    def stream_tail_store(self, h, state, batch):
        """The rows of `h` at each sequence's last taps - 1 positions into its ring (row of
        position p at p modulo taps - 1)."""
        check(self.lib.mb_stream_tail_store(
            _ptr(h), _ptr(state), state.stride(0), state.shape[1], _ptr(batch.q_start),
            _ptr(batch.kv_len), _ptr(batch.slots), batch.num_seqs, h.shape[1], self._stream()),
            "stream_tail_store")
        self.launches += 1

    # ------------------------------------------------------------------ sigmoid attention

    @_timed("rotary + store")
    def qk_norm_rope_store(self, pre, layout, q_norm, k_norm, eps, tables, pairing, batch, cache, q,
                           values_from_keys):
        """pre = [q | k (| v)] float32: per-head RMS norms of q and k (weights float32, or None),
        the rotation of their first numbers, q into `q`, keys and values into the pages; with
        `values_from_keys` the values are the keys as projected."""
        heads, kv_heads, dim, vdim = layout
        self._check_limits(cache, tables)
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        if q.dtype != cache.k.dtype:
            raise KernelError("qk_norm_rope_store: pages and activations differ in dtype")
        check(self.lib.mb_qk_norm_rope_store(
            _ptr(pre), pre.shape[1], _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(cos), _ptr(sin), rot,
            int(pairing == "interleaved"), _ptr(batch.positions), _ptr(batch.seq_of_token),
            _ptr(cache.table), cache.table.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(q), heads,
            kv_heads, dim, vdim, int(bool(values_from_keys)), cache.page_size, pre.shape[0],
            _flag(q.dtype), self._stream()), "qk_norm_rope_store")
        self.launches += 1

    @_timed("attention")
    def sigmoid_attention(self, q, layout, batch, cache, scale, window, keep_first, head_bias, out,
                          kernel: str | None = None):
        """out_h = sum over the seen keys of sigmoid(q_h . k * scale + head_bias[h]) v; key j is
        seen from position p iff j <= p and (p - j < window or j < keep_first) (window 0: all).
        `kernel` forces "mma" or "simt"; by default prompt portions in bfloat16 with a head size
        of 64 or 128 run on the tensor cores, everything else on the CUDA cores."""
        heads, kv_heads, dim, vdim = layout
        if vdim != dim:
            raise KernelError("sigmoid_attention: values of another size than the keys are not built")
        self._check_limits(cache)
        tokens = q.shape[0]
        group = heads // kv_heads
        mma_ok = q.dtype == torch.bfloat16 and bool(self.lib.mb_sigmoid_attention_mma_supports(dim))
        if kernel == "mma" and not mma_ok:
            raise KernelError(f"the tensor-core sigmoid attention takes bfloat16 with head size 64 or "
                              f"128, not {q.dtype} with {dim}")
        use_mma = mma_ok and (kernel == "mma" or (kernel is None and batch.max_q_len * group >= 64))
        rows, keys = (64, 64) if use_mma else (16, 32)
        # the keys a row looks at are bounded by the window; divide them when the batch alone
        # cannot fill the device
        if getattr(batch, "attention_splits", None):
            splits = batch.attention_splits
        else:
            reach = batch.max_kv_len if not window else min(batch.max_kv_len,
                                                           window + keep_first + batch.max_q_len)
            tiles = -(-batch.max_q_len * group // rows)
            blocks = batch.num_seqs * tiles * kv_heads
            key_tiles = -(-reach // keys)
            splits = 1
            if blocks < self.sm_count and key_tiles >= 4:
                splits = max(1, min(key_tiles // 2, -(-2 * self.sm_count // blocks), 64))
        floats = self.lib.mb_sigmoid_attention_scratch_floats(tokens, heads, dim, splits)
        scratch = self._scratch_for(floats) if floats else None
        common = (_ptr(q), _ptr(cache.k), _ptr(cache.v), _ptr(cache.table), cache.table.shape[1],
                  _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(batch.seq_of_token), _ptr(head_bias),
                  _ptr(out), _ptr(scratch), scratch.numel() if scratch is not None else 0, tokens,
                  batch.num_seqs, batch.max_q_len, heads, kv_heads, dim, cache.page_size, float(scale),
                  int(window), int(keep_first), splits)
        if use_mma:
            check(self.lib.mb_sigmoid_attention_mma(*common, self._stream()), "sigmoid_attention (mma)")
        else:
            check(self.lib.mb_sigmoid_attention(*common, _flag(q.dtype), self._stream()),
                  "sigmoid_attention")
        self.launches += 1 if splits == 1 else 2

    # ------------------------------------------------------------------ masked attention

    MASK_KINDS = {"full": 0, "sliding": 1, "chunked": 2}

    @_timed("rotary + store")
    def masked_prepare(self, pre, layout, q_norm, k_norm, eps, tables, pairing, batch, cache, q,
                       values_from_keys):
        """pre = [q | k (| v)] float32, layout (heads, kv_heads, maps, dim, vdim): one RMS norm over
        all of q's rows and one over all of k's (weights float32 over the whole projection, or
        None), the rotation of the first numbers of every map of every head, q into `q`, keys
        and values into the pages; with `values_from_keys` the values are the keys as projected."""
        heads, kv_heads, maps, dim, vdim = layout
        self._check_limits(cache, tables)
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        if q.dtype != cache.k.dtype or cache.v.dtype != cache.k.dtype:
            raise KernelError("masked_prepare: pages and activations differ in dtype")
        check(self.lib.mb_masked_prepare(
            _ptr(pre), pre.shape[1], _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(cos), _ptr(sin), rot,
            int(pairing == "interleaved"), _ptr(batch.positions), _ptr(batch.seq_of_token),
            _ptr(cache.table), cache.table.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(q), heads,
            kv_heads, maps, dim, vdim, int(bool(values_from_keys)), cache.page_size, pre.shape[0],
            _flag(q.dtype), self._stream()), "masked_prepare")
        self.launches += 1

    @_timed("attention")
    def masked_attention(self, q, layout, batch, cache, scale, mask, out, softcap=0.0, sinks=None,
                         lam=0.0, sub_eps=0.0, out_scale=1.0, kernel: str | None = None):
        """Softmax attention under `mask` = (kind, size, keep_first), kind "full", "sliding" or
        "chunked": position p sees j <= p with j >= lo(p) or j < keep_first, lo(p) = 0, p - size +
        1 or floor(p / size) * size. Scores q . k * scale, under softcap * tanh(. / softcap) when
        softcap > 0; `sinks` [heads] float32 join the denominators. With maps = 2 in the layout
        (heads, kv_heads, maps, dim, vdim) a head is two maps over the same values and its
        output (a1 - lam a2) / rms(.) * out_scale (`sub_eps` inside the root)."""
        heads, kv_heads, maps, dim, vdim = layout
        kind, size, keep_first = mask
        self._check_limits(cache)
        tokens = q.shape[0]
        group = heads // kv_heads
        # prompt portions in bfloat16 with key and value sizes the tensor-core kernel takes run
        # there (`kernel` forces "mma" or "simt"); everything else on the CUDA cores
        mma_ok = (q.dtype == torch.bfloat16
                  and bool(self.lib.mb_masked_attention_mma_supports(maps, dim, vdim)))
        if kernel == "mma" and not mma_ok:
            raise KernelError(f"the tensor-core masked attention takes bfloat16 with key and value "
                              f"sizes of 64 or 128, not {q.dtype} with {maps} x {dim} and {vdim}")
        # (decode steps too: few of a tile's 64 rows are live there, but its keys and values come
        # by 16-byte asynchronous copies two tiles deep, which is what a decode step waits for)
        use_mma = mma_ok and kernel in (None, "mma")
        rows, keys = (64, 64) if use_mma else (16, 32)
        if getattr(batch, "attention_splits", None):
            splits = batch.attention_splits
        else:
            reach = batch.max_kv_len if kind == "full" else min(
                batch.max_kv_len, size + keep_first + batch.max_q_len)
            tiles = -(-batch.max_q_len * group // rows)
            blocks = batch.num_seqs * tiles * kv_heads
            key_tiles = -(-reach // keys)
            splits = 1
            if blocks < self.sm_count and key_tiles >= 4:
                splits = max(1, min(key_tiles // 2, -(-2 * self.sm_count // blocks), 64))
        floats = self.lib.mb_masked_attention_scratch_floats(tokens, heads, maps, vdim, splits)
        scratch = self._scratch_for(floats) if floats else None
        common = (_ptr(q), _ptr(cache.k), _ptr(cache.v), _ptr(cache.table), cache.table.shape[1],
                  _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(batch.seq_of_token), _ptr(sinks),
                  _ptr(out), _ptr(scratch), scratch.numel() if scratch is not None else 0, tokens,
                  batch.num_seqs, batch.max_q_len, heads, kv_heads, maps, dim, vdim, cache.page_size,
                  float(scale), float(softcap), self.MASK_KINDS[kind], int(size), int(keep_first),
                  float(lam), float(sub_eps), float(out_scale), splits)
        if use_mma:
            check(self.lib.mb_masked_attention_mma(*common, self._stream()), "masked_attention (mma)")
        else:
            check(self.lib.mb_masked_attention(*common, _flag(q.dtype), self._stream()),
                  "masked_attention")
        self.launches += 1 if splits == 1 else 2

    # ------------------------------------------------------------------ retention

    @_timed("recurrence")
    def retention_scan(self, pre, offsets, decay, key_scale, layout, tables, pairing, cells, batch, o):
        """Per head S <- decay_h S + k v^T, o = S^T q, with q and k rotated by the token's position
        (`tables`, or None) and k then times `key_scale`; q, k and v are read off `pre` (float32) at
        `offsets`; `cells` [slots, heads * vdim * dim] float32 holds the matrices column by column;
        `o` [tokens, heads * vdim] float32."""
        heads, dim, vdim = layout
        at_q, at_k, at_v = offsets
        if pre.dtype != torch.float32 or o.dtype != torch.float32 or cells.dtype != torch.float32:
            raise KernelError("retention_scan: inputs, matrices and read-outs are float32")
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        if tables is not None:
            self._check_limits(None, tables)
        check(self.lib.mb_retention_scan(
            _ptr(pre), pre.shape[1], int(at_q), int(at_k), int(at_v), _ptr(decay), float(key_scale),
            _ptr(cos), _ptr(sin), rot, int(pairing == "interleaved"), _ptr(batch.positions),
            _ptr(cells), cells.stride(0), _ptr(batch.q_start), _ptr(batch.slots), _ptr(o),
            batch.num_seqs, heads, dim, vdim, self._stream()), "retention_scan")
        self.launches += 1

    # ------------------------------------------------------------------ latent attention

    @_timed("rotary + store")
    def latent_norm_store(self, pre, offset, rank, weight, eps, batch, cache):
        """c = rmsnorm(pre[:, offset : offset + rank]) * weight into the pages (one shared head
        of size `rank`)."""
        self._check_limits(cache)
        check(self.lib.mb_latent_norm_store(
            _ptr(pre), pre.shape[1], int(offset), _ptr(weight), _flag(weight.dtype), float(eps),
            _ptr(batch.positions), _ptr(batch.seq_of_token), _ptr(cache.table), cache.table.shape[1],
            _ptr(cache.k), int(rank), cache.page_size, pre.shape[0], _flag(cache.k.dtype),
            self._stream()), "latent_norm_store")
        self.launches += 1

    @_timed("rotary + store")
    def latent_prepare(self, pre, q_rank, q_norm, narrow, kv_offset, rank, down_norm, rot_dim, tables,
                       pairing, eps, batch, cache):
        """narrow = rmsnorm(pre[:, :q_rank]) * q_norm (if q_rank); with a cache, the row [c | rotated
        part] of every token into its page: c = rmsnorm(pre[:, kv_offset : kv_offset + rank]) *
        down_norm, the part pre[:, kv_offset + rank : + rot_dim] rotated by the token's position."""
        if cache is not None:
            self._check_limits(cache, tables)
        cos, sin = tables if tables is not None else (None, None)
        weights = [w for w in (q_norm, down_norm) if w is not None]
        if len({w.dtype for w in weights}) > 1:
            raise KernelError("latent_prepare: the two norm weights differ in dtype")
        kind = narrow if narrow is not None else (cache.k if cache is not None else None)
        if kind is None:
            return
        if narrow is not None and cache is not None and narrow.dtype != cache.k.dtype:
            raise KernelError("latent_prepare: pages and activations differ in dtype")
        check(self.lib.mb_latent_prepare(
            _ptr(pre), pre.shape[1], int(q_rank), _ptr(q_norm), _ptr(narrow), int(kv_offset), int(rank),
            _ptr(down_norm), _flag(weights[0].dtype) if weights else 0, int(rot_dim), _ptr(cos),
            _ptr(sin), int(pairing == "interleaved"), float(eps), _ptr(batch.positions),
            _ptr(batch.seq_of_token), _ptr(cache.table) if cache is not None else None,
            cache.table.shape[1] if cache is not None else 0,
            _ptr(cache.k) if cache is not None else None,
            cache.page_size if cache is not None else 1, pre.shape[0], _flag(kind.dtype),
            self._stream()), "latent_prepare")
        self.launches += 1

    @_timed("rotary + store")
    def rope_rows(self, q, heads, row, offset, rot_dim, tables, pairing, batch):
        """In place: q[t, h * row + offset : + rot_dim] rotated by the token's position."""
        cos, sin = tables
        check(self.lib.mb_rope_rows(
            _ptr(q), _flag(q.dtype), int(heads), int(row), int(offset), int(rot_dim), _ptr(cos),
            _ptr(sin), int(pairing == "interleaved"), _ptr(batch.positions),
            _ptr(batch.seq_of_token), q.shape[0], self._stream()), "rope_rows")
        self.launches += 1

    @_timed("head product")
    def head_linear(self, x, offset, weight, out):
        """out[t, h] = weight[h]^T x[t, h]: weight [heads, in, out] (input-major), x's heads
        side by side from column `offset`."""
        heads, cols, outs = weight.shape
        self._rows(weight)
        tokens = x.shape[0]
        if (self.head_product_library and weight.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and tokens >= self.head_product_library_min_tokens and cols % 8 == 0 and outs % 8 == 0
                and offset % 8 == 0 and x.shape[1] % 8 == 0):
            # many tokens in bfloat16: one batched product of the library over the heads, read
            # and written in place through strided views (the engine's other many-token
            # products are the library's too)
            rows = x[:, offset:offset + heads * cols]
            if rows.dtype != torch.bfloat16:
                rows = rows.to(torch.bfloat16)
            torch.bmm(rows.view(tokens, heads, cols).transpose(0, 1), weight,
                      out=out.view(tokens, heads, outs).transpose(0, 1))
            self.library_calls += 1
            return
        check(self.lib.mb_head_linear(
            _ptr(x), _flag(x.dtype), x.shape[1], int(offset), _ptr(weight), _flag(weight.dtype),
            _ptr(out), _flag(out.dtype), x.shape[0], heads, cols, outs, self._stream()), "head_linear")
        self.launches += 1

    # ------------------------------------------------------------------ routed experts

    @_timed("router")
    def route_experts(self, x, router, correction, group_count, group_keep, route_scale, chosen,
                      weights):
        if self._pending(x) is not None:
            x = x.materialize()
        tokens, top = chosen.shape
        experts = router.shape[0]
        if self._router_logits is None or self._router_logits.numel() < tokens * experts:
            if self._router_logits is not None:
                self._retired.append(self._router_logits)    # captured graphs still write there
            self._router_logits = torch.empty(max(tokens * experts, 1 << 16), dtype=torch.float32,
                                              device=self.device)
        check(self.lib.mb_route_experts(
            _ptr(x), _flag(x.dtype), _ptr(router), _ptr(correction), _ptr(self._router_logits),
            _ptr(chosen), _ptr(weights), tokens, x.shape[1], experts, top, int(group_count),
            int(group_keep), float(route_scale), self._stream()), "route_experts")
        fused = tokens <= 32 and (x.shape[1] + 5 * experts) * 4 <= 48 * 1024
        self.launches += 1 if fused else 2

    @_timed("expert products")
    def expert_feed_forward(self, x, chosen, weights, gate_up, down, out, ctx, weight_on="output"):
        """out[t] = sum_j weights[t, j] * down[e] (silu(gate[e] x[t]) * (up[e] x[t])), e =
        chosen[t, j]: the step's (token, choice) pairs sorted by expert, two grouped products,
        and the weighted sum in the order of the choice. `weight_on` "input": the weight
        multiplies what the expert reads instead, out[t] = sum_j expert_e(weights[t, j] x[t]); the
        experts have no biases, so the weight is applied to both first products' results (or to
        the gathered rows, where the library multiplies) and the sum is unweighted."""
        if self._pending(x) is not None:
            x = x.materialize()
        tokens, top = chosen.shape
        experts, _two_ff, hidden = gate_up.shape
        ff = down.shape[2]
        pairs = tokens * top
        # rows per tile: 128 on the tensor cores (bfloat16, sizes in multiples of 8), else 32
        bm = self.lib.mb_expert_tile_rows(_flag(x.dtype), hidden, ff) if self.expert_tensor_cores else 32
        cap = self.lib.mb_expert_tile_cap(pairs, experts, bm)
        plan = ctx.buffer("expert_plan", 1 + 3 * cap + 2 * pairs + experts, 1, dtype=torch.int32)
        check(self.lib.mb_expert_plan(_ptr(chosen), pairs, experts, cap, bm, _ptr(plan),
                                      self._stream()), "expert_plan")
        if (self.expert_library and self._grouped_mm is not None and x.dtype == torch.bfloat16
                and gate_up.dtype == torch.bfloat16 and down.dtype == torch.bfloat16
                and pairs >= self.expert_library_min_pairs and hidden % 8 == 0 and ff % 8 == 0):
            return self._expert_library(x, weights, gate_up, down, out, ctx, plan, cap, tokens, top,
                                        weight_on)
        act = ctx.buffer("expert_act", pairs, ff)
        if act.dtype != x.dtype or gate_up.dtype != x.dtype or down.dtype != x.dtype:
            raise KernelError("expert_feed_forward: activations and expert matrices differ in dtype")
        on_input = weight_on == "input"
        check(self.lib.mb_expert_product(0, _ptr(x), x.shape[1], _ptr(gate_up), _ptr(act), _ptr(plan),
                                         cap, top, hidden, ff, _flag(x.dtype), bm,
                                         _ptr(weights) if on_input else None, self._stream()),
              "expert gate/up product")
        y = ctx.buffer("expert_rows", pairs, hidden, dtype="float32")
        check(self.lib.mb_expert_product(1, _ptr(act), ff, _ptr(down), _ptr(y), _ptr(plan), cap, top,
                                         ff, hidden, _flag(x.dtype), bm, None, self._stream()),
              "expert down product")
        check(self.lib.mb_expert_combine(_ptr(y), None if on_input else _ptr(weights), _ptr(out),
                                         tokens, top, hidden,
                                         self._stream()), "expert_combine")
        self.launches += 4

    def _expert_library(self, x, weights, gate_up, down, out, ctx, plan, cap, tokens, top,
                        weight_on="output"):
        """Many pairs in bfloat16: the two grouped products are the library's (where the
        engine's other many-token products are the library's too), between this package's
        gather, gate and weighted sum. The rows lie in the plan's order throughout."""
        experts, _two_ff, hidden = gate_up.shape
        ff = down.shape[2]
        pairs = tokens * top
        flat = plan.view(-1)
        perm = flat[1 + 3 * cap:1 + 3 * cap + pairs]
        ends = flat[1 + 3 * cap + pairs:1 + 3 * cap + pairs + experts]
        place = flat[1 + 3 * cap + pairs + experts:]
        rows = ctx.buffer("expert_in", pairs, hidden)
        on_input = weight_on == "input"
        check(self.lib.mb_expert_gather(_ptr(x), _ptr(perm), _ptr(rows), pairs, top, hidden,
                                        _ptr(weights) if on_input else None, self._stream()),
              "expert_gather")
        both = self._grouped_mm(rows, gate_up.transpose(1, 2), offs=ends)
        act = ctx.buffer("expert_act", pairs, ff)
        self.swiglu(both, act)
        y = self._grouped_mm(act, down.transpose(1, 2), offs=ends)
        check(self.lib.mb_expert_combine_sorted(_ptr(y), _ptr(place),
                                                None if on_input else _ptr(weights), _ptr(out), tokens,
                                                top, hidden, self._stream()), "expert_combine")
        self.launches += 3
        self.library_calls += 2

    # ------------------------------------------------------------------ mixed-head attention

    @_timed("rotary + store")
    def rope_blend_store(self, qkv, layout, tables, batch, cache, blend_from, blend, keep):
        """Packed rows [q | k | v] with heads of (dim, dim, vdim): rotate the leading features
        of q and k, copy v to `keep`, blend v with `blend_from` by the device scalar `blend`,
        store k and v into the pages."""
        heads, kv_heads, dim, vdim = layout
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        self._check_limits(cache, tables)
        if cache.k.dtype != qkv.dtype:
            raise KernelError("rope_blend_store: pages and activations differ in dtype")
        check(self.lib.mb_rope_blend_store(
            _ptr(qkv), _ptr(cos), _ptr(sin), rot, _ptr(batch.positions), _ptr(batch.seq_of_token),
            _ptr(cache.table), cache.table.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(blend_from),
            _ptr(blend), _ptr(keep), qkv.shape[0], heads, kv_heads, dim, vdim, cache.page_size,
            int(cache.write), _flag(qkv.dtype), self._stream()), "rope_blend_store")
        self.launches += 1

    @_timed("attention")
    def mixed_head_attention(self, qkv, layout, batch, cache, scale, window, mix, out,
                             kernel: str | None = None):
        """Attention over the pages whose heads' softmax weights are mixed by `mix`
        [heads, heads] (float32, or None) before they meet the values. bfloat16 with sizes
        the tensor-core kernel takes runs there (`kernel` forces "mma" or "simt"), everything
        else, and the float32 engine always, on the CUDA cores."""
        heads, kv_heads, dim, vdim = layout
        self._check_limits(cache)
        tokens = qkv.shape[0]
        mma_ok = (qkv.dtype == torch.bfloat16 and qkv.shape[1] % 8 == 0
                  and bool(self.lib.mb_mixed_head_mma_supports(heads, kv_heads, dim, vdim)))
        if kernel == "mma" and not mma_ok:
            raise KernelError("the tensor-core mixed-head attention takes bfloat16, heads of a "
                              "multiple of 16 features and value heads of a multiple of 8 up to 128")
        use_mma = mma_ok and (kernel or self.mixed_head) != "simt"
        splits = self._mixed_head_splits(batch, heads, 16 if use_mma else None)
        floats = self.lib.mb_mixed_head_scratch_floats(tokens, heads, vdim, splits)
        scratch = self._scratch_for(floats) if floats else None
        if use_mma:
            check(self.lib.mb_mixed_head_attention_mma(
                _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
                cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(mix), _ptr(out),
                batch.num_seqs, batch.max_q_len, heads, kv_heads, dim, vdim, cache.page_size,
                float(scale), int(window), splits, _ptr(batch.seq_of_token), tokens, _ptr(scratch),
                scratch.numel() if scratch is not None else 0, self._stream()),
                "mixed_head_attention (mma)")
            self.launches += 1 if splits == 1 else 3
            return
        check(self.lib.mb_mixed_head_attention(
            _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
            cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(mix), _ptr(out),
            batch.num_seqs, batch.max_q_len, heads, kv_heads, dim, vdim, cache.page_size,
            float(scale), int(window), _flag(qkv.dtype), splits, _ptr(batch.seq_of_token), tokens,
            _ptr(scratch), scratch.numel() if scratch is not None else 0, self._stream()),
            "mixed_head_attention")
        self.launches += 1 if splits == 1 else 3

    def _mixed_head_splits(self, batch, heads: int, rows: int | None = None) -> int:
        """Key ranges per row tile of the mixed-head attention. One block holds every head of
        a tile of tokens, so a step brings few blocks (one per sequence when decoding, 128
        for a 2048-token prompt on the tensor-core kernel) and the longest of them walks
        every key twice: the keys are divided until the device holds about
        `mixed_head_blocks_per_sm` blocks per SM, at most `mixed_head_max_splits` ways.
        Inside a captured step (the batch names `attention_splits`) the count depends on the
        batch's shape only, never on its lengths; a block whose range is empty leaves zeros.
        `rows`: tokens per block of the tensor-core kernel (the CUDA-core kernel's follow
        from the head count)."""
        if self.decode_splits is not None:
            return max(1, self.decode_splits)
        bq = rows or max(1, min(64 // heads, 16, batch.max_q_len))
        blocks = batch.num_seqs * -(-batch.max_q_len // bq)
        # one row tile a sequence (a decode step): every block is as heavy as the others and
        # the tensor-core kernel keeps one block on an SM, so one wave is the aim
        per_sm = 1 if rows and batch.max_q_len <= rows else self.mixed_head_blocks_per_sm
        fill = max(1, min(self.mixed_head_max_splits, per_sm * self.sm_count // blocks))
        if getattr(batch, "attention_splits", None):
            return fill
        key_tiles = -(-batch.max_kv_len // 32)
        return max(1, min(fill, key_tiles // 2))

    def qkv_rope_store(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables,
                       batch, cache):
        """The packed q/k/v projection with bias, then rotation of q and k and the store of
        k and v into the cache pages: one kernel for few tokens, two otherwise."""
        m, k = x.shape
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        self._check_limits(cache, tables)
        if (self.skinny and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and (bias is None or bias.dtype == torch.bfloat16) and cache is not None
                and cache.k.dtype == torch.bfloat16
                and self.lib.mb_gemm_skinny_qkv_supports(m, k, head_dim, rot)):
            self._qkv_rope_fused(x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, cos, sin,
                                 rot, batch, cache)
            return
        if self._pending(x) is not None:
            x = x.materialize()
        with self._as("q/k/v product"):
            self.linear(x, weight, bias, qkv)
        self.rope_cache_write(qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache)

    @_timed("q/k/v + rotary + store")
    def _qkv_rope_fused(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, cos, sin, rot,
                        batch, cache):
        m, k = x.shape
        xp, hp, wp, _rows, eps, ssp, sst, sse, ssk = self._skinny_input(x)
        check(self.lib.mb_gemm_skinny_qkv_rope(
            xp, hp, wp, eps, ssp, sst, sse, ssk, _ptr(weight), _ptr(bias), _ptr(qkv), _ptr(cos), _ptr(sin), rot,
            _ptr(batch.positions), _ptr(batch.seq_of_token), _ptr(cache.table),
            cache.table.shape[1], _ptr(cache.k), _ptr(cache.v), m, k, num_heads, num_kv_heads,
            head_dim, cache.page_size, int(cache.write), self._stream()),
            "qkv_rope_store (skinny)")
        self.launches += 1

    @_timed("gate")
    def swiglu(self, gate_up, out):
        check(self.lib.mb_swiglu(_ptr(gate_up), _ptr(out), out.shape[0], out.shape[1],
                                 _flag(out.dtype), self._stream()), "swiglu")
        self.launches += 1

    @_timed("rotary + store")
    def rope_cache_write(self, qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache):
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        store = int(cache is not None and cache.write)
        self._check_limits(cache, tables)
        if cache is not None and cache.k.dtype != qkv.dtype:
            raise KernelError("rope_cache_write: pages and activations differ in dtype")
        check(self.lib.mb_rope_store(
            _ptr(qkv), _ptr(cos), _ptr(sin), rot, _ptr(batch.positions),
            _ptr(batch.seq_of_token), _ptr(cache.table) if cache is not None else None,
            cache.table.shape[1] if cache is not None else 0,
            _ptr(cache.k) if cache is not None else None,
            _ptr(cache.v) if cache is not None else None,
            qkv.shape[0], num_heads, num_kv_heads, head_dim,
            cache.page_size if cache is not None else 1, store, _flag(qkv.dtype),
            self._stream()), "rope_cache_write")
        self.launches += 1

    def _splits(self, batch, num_kv_heads, group, rows_per_block, keys_per_tile) -> int:
        """Divide the keys over more blocks when the batch alone cannot fill the device."""
        if getattr(batch, "attention_splits", None):
            return batch.attention_splits
        if self.decode_splits is not None:
            return max(1, self.decode_splits)
        tiles = -(-batch.max_q_len * group // rows_per_block)
        blocks = batch.num_seqs * tiles * num_kv_heads
        key_tiles = -(-batch.max_kv_len // keys_per_tile)
        if blocks >= self.sm_count or key_tiles < 4:
            return 1
        return max(1, min(key_tiles // 2, -(-2 * self.sm_count // blocks), 64))

    def graph_splits(self, sequences: int, num_kv_heads: int) -> int:
        """How many ways the keys of each sequence are split in a captured decode step of
        `sequences` rows: sized to fill the device whatever the lengths turn out to be."""
        if self.decode_splits:
            return max(1, int(self.decode_splits))
        rows = max(1, sequences * num_kv_heads)
        if rows <= self.graph_small_rows:
            return max(1, min(self.graph_max_ranges_small,
                              self.graph_blocks_per_sm_small * self.sm_count // rows))
        return max(1, -(-self.graph_blocks_per_sm_large * self.sm_count // rows))

    def _prompt_cluster(self, batch, num_kv_heads, group) -> int:
        """CTAs per row tile of the tensor-memory attention: the CTAs of a cluster share a
        row tile and split its keys (merged through distributed shared memory). It pays only
        while the row tiles alone leave SMs idle, that is for portions of a prompt: measured
        on B200 (14 heads over 2 KV heads of 64, context 2048, replayed from a graph) a prompt
        in portions of 256 tokens (30 row tiles a step) took 11.3 ms whole, 10.7 ms in pairs and
        10.5 in fours; in portions of 512 (58 row tiles) 6.13 and 6.13 ms; in one step of 2048
        tokens (228 row tiles) 2.8 ms whole, 3.5 in pairs, 4.5 in fours."""
        if self.prompt_cluster is not None:
            return self.prompt_cluster
        tokens_per_tile = max(1, 128 // group)
        row_tiles = batch.num_seqs * -(-batch.max_q_len // tokens_per_tile) * num_kv_heads
        if batch.max_kv_len < 4 * 128:
            return 1
        cluster = 1
        while cluster < 4 and row_tiles * cluster * 2 <= self.sm_count:
            cluster *= 2
        return cluster

    def _prompt_splits(self, batch, num_kv_heads, group) -> int:
        """Key ranges per row tile of a prompt portion. Cutting the keys (and merging the
        ranges afterwards) shortens the chain of the last, heaviest row tile, but on B200 a
        2048-token portion got slower with every cut (3.87 ms whole, 4.09 ms in two, 4.43 ms
        in eight: the float32 partial results cost more than the tail), so prompts are not
        cut unless `prompt_splits` says so."""
        if self.prompt_splits is not None:
            return max(1, self.prompt_splits)
        return 1

    @_timed("attention")
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                        window, out, kernel: str | None = None, sinks=None):
        """`kernel` forces "mma" or "simt"; by default bfloat16 with a head size the
        tensor-core kernel takes runs there, everything else on the CUDA cores. `sinks`
        (float32, one per query head): exp(sink) joins the softmax's denominator."""
        group = num_heads // num_kv_heads
        tokens = qkv.shape[0]
        self._check_limits(cache)
        tc_ok = (qkv.dtype == torch.bfloat16 and self.lib.mb_attention_tcgen05_supports(
            head_dim, cache.page_size, num_heads, num_kv_heads, qkv.shape[1]))
        if kernel == "tcgen05" and not tc_ok:
            raise KernelError("the tensor-memory attention takes bfloat16, head sizes 64 and 128 and "
                              "pages of 8 to 128 tokens")
        # prompt portions (at least one full tile of rows) go to the tensor-memory kernel
        if tc_ok and (kernel == "tcgen05" or (kernel is None and self.attention == "auto"
                                              and batch.max_q_len * group >= 128)):
            check(self.lib.mb_paged_attention_tcgen05(
                _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), cache.k.shape[0],
                _ptr(cache.table), cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len),
                _ptr(out), tokens, batch.num_seqs, batch.max_q_len, num_heads, num_kv_heads,
                head_dim, cache.page_size, float(scale), int(window),
                self._prompt_cluster(batch, num_kv_heads, group), _ptr(self._error_word()),
                _ptr(sinks), self._stream()), "paged_attention (tcgen05)")
            self.launches += 1
            self._tc_pending = True
            return
        use_mma = (qkv.dtype == torch.bfloat16 and self.lib.mb_attention_mma_supports(head_dim)
                   and kernel != "simt")
        if kernel == "mma" and not use_mma:
            raise KernelError(f"the tensor-core attention takes bfloat16 with head size 64 or "
                              f"128, not {qkv.dtype} with {head_dim}")
        if use_mma:
            small = batch.max_q_len * group <= 16
            if small:
                splits = self._splits(batch, num_kv_heads, group, 16, 64)
                if self.decode_clusters and splits < 32 and kernel is None and cache.page_size >= 2:
                    cluster = self._cluster_of(splits)
                    self._decode_cluster(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                                         window, out, cluster, None, False, sinks)
                    return
                if sinks is not None:
                    # so many key ranges that they meet in global memory: the CUDA-core kernel
                    use_mma = False
                    splits = self._splits(batch, num_kv_heads, group, 16, 32)
            else:
                splits = self._prompt_splits(batch, num_kv_heads, group)
        else:
            splits = self._splits(batch, num_kv_heads, group, 16, 32)
        if sinks is not None and not use_mma:
            return self._attention_with_sinks(qkv, num_heads, num_kv_heads, head_dim, batch, cache,
                                              scale, window, out, sinks, splits)
        floats = self.lib.mb_attention_scratch_floats(tokens, num_heads, head_dim, splits)
        scratch = self._scratch_for(floats) if floats else None
        common = (_ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
                  cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len),
                  _ptr(batch.seq_of_token), _ptr(out), _ptr(scratch),
                  scratch.numel() if scratch is not None else 0, tokens, batch.num_seqs,
                  batch.max_q_len, num_heads, num_kv_heads, head_dim, cache.page_size, float(scale),
                  int(window), splits)
        if use_mma:
            counters = None
            if splits > 1 and small:
                counters = self._counters_for(batch.num_seqs * num_kv_heads)
            check(self.lib.mb_paged_attention_mma_sinks(*common, _ptr(counters), _ptr(sinks),
                                                        self._stream()), "paged_attention (mma)")
            self.launches += 1 if (splits == 1 or counters is not None) else 2
            return
        else:
            check(self.lib.mb_paged_attention_simt(*common, _flag(qkv.dtype), self._stream()),
                  "paged_attention")
        self.launches += 1 if splits == 1 else 2

    def _attention_with_sinks(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                              window, out, sinks, splits):
        """The CUDA-core kernel with sinks: the float32 engine, and bfloat16 sizes the
        tensor-core kernels refuse."""
        tokens = qkv.shape[0]
        floats = self.lib.mb_attention_scratch_floats(tokens, num_heads, head_dim, splits)
        scratch = self._scratch_for(floats) if floats else None
        check(self.lib.mb_paged_attention_simt_sinks(
            _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
            cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(batch.seq_of_token),
            _ptr(out), _ptr(scratch), scratch.numel() if scratch is not None else 0, tokens,
            batch.num_seqs, batch.max_q_len, num_heads, num_kv_heads, head_dim, cache.page_size,
            float(scale), int(window), splits, _flag(qkv.dtype), _ptr(sinks), self._stream()),
            "paged_attention (sinks)")
        self.launches += 1 if splits == 1 else 2

    @_timed("attention")
    def _decode_cluster(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window,
                        out, cluster, tables, raw, sinks=None):
        cos, sin = tables if tables is not None else (None, None)
        self._check_limits(cache, tables)
        # blocks that walk many key tiles each (a large batch) get their tiles by TMA
        fed = self._long_ranges(batch, num_kv_heads, head_dim)
        if fed:
            self._tc_pending = True
        check(self.lib.mb_paged_attention_decode_cluster_sinks(
            _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
            cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(out),
            qkv.shape[0], batch.num_seqs, batch.max_q_len, num_heads, num_kv_heads, head_dim,
            cache.page_size, float(scale), int(window), cluster, _ptr(cos), _ptr(sin), int(raw),
            int(cache.write), cache.k.shape[0] if fed else 0, _ptr(self._error_word()) if fed else None,
            _ptr(sinks), self._stream()), "paged_attention (decode clusters)")
        self.launches += 1

    def _long_ranges(self, batch, num_kv_heads, head_dim=64) -> bool:
        """Whether the cluster decode kernel takes its TMA-fed form. Head size 64: when its
        blocks will walk many key tiles each, that is when the batch alone brings more
        (sequence, KV head) pairs than `graph_small_rows`, so that few key ranges per pair fill
        the device (for small batches every tile is in shared memory before the kernel in
        front is done, and 16 bytes per thread and copy are the faster way there). Head size
        128, whose tiles cost a thread twice the copies: from 16 pairs on (measured on B200
        inside the captured decode step, 1.5B sizes: 8 sequences 1.56 -> 1.34 ms, 16: 2.10 ->
        1.76; 4 sequences 1.23 -> 1.25, one 1.18 -> 1.22)."""
        if self.decode_long_ranges is not None:
            return bool(self.decode_long_ranges)
        pairs = batch.num_seqs * num_kv_heads
        if head_dim > 64:
            return pairs >= self.graph_small_rows
        return pairs > 2 * self.graph_small_rows

    @staticmethod
    def _cluster_of(splits: int) -> int:
        cluster = 1
        while cluster * 2 <= min(splits, 8):
            cluster *= 2
        return cluster

    def qkv_attention(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables, batch,
                      cache, scale, window, out):
        """Projection of q/k/v, rotation, store of the new keys and values, and attention over
        the cache. For decode-like batches (bfloat16, head size 64 or 128, whole-head rotation
        or none) the projection is the plain product for that many tokens (few tokens: as many
        blocks as row tiles, where the fused q/k/v kernel has one per head; more: the
        library's, and the rotary/store kernel's launch is saved), and the attention kernel rotates the
        queries as it loads them and rotates and stores the new keys itself; otherwise
        `qkv_rope_store` followed by `paged_attention`. Measured on B200 inside the captured
        decode step (2048-token contexts): Qwen2.5-0.5B sizes, head size 64: batch 8 0.671 ->
        0.660 ms, batch 1 0.667 -> 0.633 ms, batch 16 1.23 -> 1.11 ms, batch 32 1.27 -> 1.19 ms, batch 64 1.49 ->
        1.42 ms; head size 128: 1.5B sizes batch 16 2.18 -> 2.07 ms, 7B sizes batch 8 3.93 ->
        3.73 ms. Which head sizes gain is the kernel's to say (mb_attention_decode_raw_pays)."""
        m, k = x.shape
        group = num_heads // num_kv_heads
        cos = tables[0] if tables is not None else None
        fused = (self.decode_clusters and weight.dtype == torch.bfloat16
                 and x.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
                 and cache is not None and cache.write and cache.k.dtype == torch.bfloat16
                 and cache.page_size >= 2
                 and qkv.dtype == torch.bfloat16 and batch.max_q_len * group <= 16
                 and self.lib.mb_attention_mma_supports(head_dim)
                 and self.lib.mb_attention_decode_raw_pays(head_dim)
                 and (cos is None or 2 * cos.shape[1] == head_dim))
        splits = self._splits(batch, num_kv_heads, group, 16, 64) if fused else 0
        if not fused or splits >= 32:
            self.qkv_rope_store(x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables,
                                batch, cache)
            self.paged_attention(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window,
                                 out)
            return
        with self._as("q/k/v product"):
            self.linear(x, weight, bias, qkv)
        self._decode_cluster(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window,
                             out, self._cluster_of(splits), tables, True)

    @_timed("sampling")
    def argmax(self, logits, out):
        rows = logits.shape[0]
        if self._argmax_scratch is None or self._argmax_scratch.numel() < rows * 128:
            if self._argmax_scratch is not None:
                self._retired.append(self._argmax_scratch)
            self._argmax_scratch = torch.empty(max(rows, 64) * 128, dtype=torch.float32,
                                               device=self.device)
        check(self.lib.mb_argmax(_ptr(logits), _ptr(out), rows, logits.shape[1],
                                 _ptr(self._argmax_scratch), self._stream()), "argmax")
        self.launches += 2 if logits.shape[1] >= 16384 else 1

    @_timed("sampling")
    def sample(self, logits, temperature, top_p, u, out):
        check(self.lib.mb_sample(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(u), _ptr(out),
                                 logits.shape[0], logits.shape[1], self._stream()), "sample")
        self.launches += 1
