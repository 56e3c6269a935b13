"""The CUDA kernel set: what the parts call.

Each method checks its tensors (device, dtype, contiguity, shapes), allocates the output
with torch and launches a hand-written kernel of the library on torch's current stream.
torch is the tensor container and allocator here, nothing more: no torch operator
computes anything on this path.
"""

from __future__ import annotations

import ctypes
import weakref

import torch

from . import library
from .attention_plan import KEY_CHUNK, query_tiles
from .library import KernelLibraryError, check

EPILOGUES = {"none": 0, "gelu_tanh": 1, "residual": 2}
SKINNY_ROWS = 16         # most tokens the small-batch projection kernel takes
CLUSTER_ROWS = 128       # most tokens the mid-batch (K split over a cluster) projection kernel takes
CLUSTER_WIDE_MAX_BYTES = 3 << 20   # ... and the largest matrix it is given for more than 64 tokens
PREFETCH_MAX_BYTES = 32 << 20   # most of a following matrix that a streaming projection asks into L2
STREAM_MIN_ROWS = 8192   # a matrix this tall (the head) goes through the streaming kernel ...
STREAM_ROWS = 16         # ... for up to this many tokens (it takes 64; beyond 16 the tensor-core GEMM measured faster)


class DeferredNorm:
    """A LayerNorm that has not run yet: the projection that consumes it may fuse it into its
    prologue (small batches) or ask for it to be materialised.  ``rows`` optionally selects
    rows of ``x32`` first."""

    def __init__(self, ops, x32, gain, shift, eps, out_dtype, rows=None) -> None:
        self.ops, self.x32, self.gain, self.shift, self.eps = ops, x32, gain, shift, float(eps)
        self.dtype, self.rows = out_dtype, rows
        self.shape = (x32.shape[0] if rows is None else rows.numel(), x32.shape[1])

    def materialize(self):
        x = self.x32 if self.rows is None else self.ops.gather_rows(self.x32, self.rows)
        return self.ops.layernorm(x, self.gain, self.shift, self.eps, self.dtype)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _ptr(t):
    return None if t is None else t.data_ptr()


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device="cuda:0") -> None:
        if not torch.cuda.is_available():
            raise KernelLibraryError(
                "no CUDA device: this engine runs only on its sm_100a kernels and has no "
                "CPU path")
        self.device = torch.device(device)
        self.index = self.device.index or 0
        self.lib = library.load()
        torch.cuda.init()
        with torch.cuda.device(self.index):
            torch.empty(1, device=self.device)      # make sure the primary context exists
        arch = self.lib.mg_device_arch(self.index)
        if arch < 0:
            check(arch, "device query")
        if arch // 10 != 10:
            raise KernelLibraryError(
                f"device {self.index} has compute capability {arch / 10:.1f}; the kernels "
                "are built for sm_100a (NVIDIA B200) only")
        check(self.lib.mg_set_device(self.index), "set device")
        self.launches = 0          # kernels launched through this object
        # a guarded build (MINIGPT_B200_GUARDS=1): the kernels check the indices they read from device memory
        self.guards = bool(self.lib.mg_guards_enabled())
        # Kernels with bounded waits record a non-zero code here if a wait ran out.
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.use_tensor_cores = True
        self.use_split_attention = True
        self.use_skinny = True
        self.use_cluster = True
        self.use_stream = True
        self.use_wide = True
        # The large-matrix kernels also take any matrix of at least `stream_min_bytes` (None: only tall
        # ones, the head).  Measured with 8 tokens: a 5.1 MB matrix (1600 x 1600) is faster through
        # the kernel of tiled copies than through the small-batch kernel, matrices of 4.7 MB (3072 x
        # 768 and its transpose) are slower by a tenth; the boundary sits between them.  Where that
        # kernel refuses, the row-streaming kernel takes over, with rows cut into up to
        # `stream_max_chunks` K chunks (at 6400 columns, 67 chunks of 192 bytes, it was measured far
        # slower than the small-batch kernel, hence the limit).
        self.stream_min_bytes = 5_000_000
        self.stream_max_chunks = 8
        self.greedy_taken = False
        self.use_dependent_launch = True
        self.use_prefill_tc = True
        self._counter_buf = None
        self._retired_counters = []
        self._sm_count = None
        self.use_fused_mlp = True
        # A streaming projection asks the weights of the projection that followed it the last time into
        # L2 once its own are on their way (learned from the order of the calls: a step repeats it).
        self.use_weight_prefetch = True
        self._last_weight = None   # data pointer of the matrix of the last projection
        self._next_weight = {}     # data pointer of a matrix -> weak reference to the matrix that came next
        self._packed = {}          # data pointer of a matrix -> (the matrix, its copy packed for a kernel)
        self._tile_lists = {}      # (rows, contexts, slots) of a step -> the prompt attention's work list
        self._ring = None          # (tensor that holds the residual stream, zeroed buffer, spare buffer)

    def begin_forward(self) -> None:
        """A forward pass begins: the first projection of a pass follows no other (the hint for the
        L2 prefetch never points from one pass, or one model, into another)."""
        self._last_weight = None

    # ---- helpers --------------------------------------------------------------------------
    def _run(self, code: int, what: str) -> None:
        """Check a launch's return code and count it."""
        check(code, what)
        self.launches += 1

    def _stream(self):
        # the raw handle of torch's current stream; the private getter costs a tenth of a
        # microsecond, building a Stream object two: it matters at sixty launches a step
        if _raw_stream is not None:
            return _raw_stream(self.index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _want(self, t, dtype, name, dims=None):
        if t.device != self.device:
            raise KernelLibraryError(f"{name}: tensor on {t.device}, kernels run on {self.device}")
        if dtype is not None and t.dtype != dtype:
            raise KernelLibraryError(f"{name}: dtype {t.dtype}, expected {dtype}")
        if not t.is_contiguous():
            raise KernelLibraryError(f"{name}: tensor must be contiguous")
        if dims is not None and t.dim() != dims:
            raise KernelLibraryError(f"{name}: expected {dims} dims, got shape {tuple(t.shape)}")
        return t

    @staticmethod
    def _is_bf16(t) -> int:
        if t.dtype == torch.bfloat16:
            return 1
        if t.dtype == torch.float32:
            return 0
        raise KernelLibraryError(f"dtype {t.dtype} is neither bfloat16 nor float32")

    def _counters(self, count: int):
        """Zeroed ints that the split attention kernel uses to find its last block per row and
        leaves zeroed; kept for the life of the object, grown on demand (a buffer that was
        handed out once is never freed)."""
        if self._counter_buf is None or self._counter_buf.numel() < count:
            if self._counter_buf is not None:
                # A captured graph may hold the old buffer's address: it stays alive (and zeroed,
                # as its kernels leave it) for as long as this object does.
                self._retired_counters.append(self._counter_buf)
            self._counter_buf = torch.zeros(max(count, 4096, 2 * (self._counter_buf.numel()
                                                                   if self._counter_buf is not None else 0)),
                                            dtype=torch.int32, device=self.device)
        return self._counter_buf

    def set_dependent_launch(self, on: bool) -> None:
        """Let kernels that support it start while the kernel before them drains (used while a
        decode step is captured into a CUDA graph)."""
        check(self.lib.mg_set_dependent_launch(1 if (on and self.use_dependent_launch) else 0),
              "set_dependent_launch")

    def check_indices(self) -> None:
        """Guarded builds: raise if a kernel met a token id, position, cache row, page, request or row
        number outside its table since the last call (synchronises; the kernel skipped the access
        or read index 0 in its place, so the results of that step are invalid but no memory
        outside a table was touched).  Ordinary builds: nothing to ask."""
        if not self.guards:
            return
        torch.cuda.synchronize(self.device)
        record = (ctypes.c_longlong * 4)()
        faults = []
        for name in library.GUARDED_FILES:
            check(getattr(self.lib, f"mg_{name}_index_fault")(record), "index guard")
            if record[0]:
                what = library.GUARD_CODES.get(int(record[0]), f"index (code {record[0]})")
                faults.append(f"{name}: {what} {record[2]} is outside 0..{record[3] - 1} (block {record[1]})")
        if faults:
            raise KernelLibraryError("a kernel met an index outside its table: " + "; ".join(faults))

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits ran out (synchronises); in a
        guarded build also if one met an index outside its table."""
        self.check_indices()
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise KernelLibraryError(f"a kernel gave up waiting (code {code}); its results are invalid")

    def wait_probe(self, limit: int = 1000) -> None:
        """Run a kernel whose bounded wait runs out (it waits ``limit`` tries on a barrier that is
        never completed, with the wait all kernels share) and records its code in the status
        word: what ``check_status`` and the engine then do can be seen without any fault."""
        self._run(self.lib.mg_wait_probe(int(limit), _ptr(self.status), self._stream()), "wait probe")

    def status_to_host(self, pinned=None):
        """Queue a copy of the status word into pinned host memory on the current stream and
        return that memory; once the stream has been synchronised (or an event recorded after
        this call has), ``raise_on_status(pinned)`` tells whether a kernel before it gave up."""
        if pinned is None:
            pinned = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        pinned.copy_(self.status, non_blocking=True)
        return pinned

    def raise_on_status(self, pinned) -> None:
        self.check_indices()
        code = int(pinned[0])
        if code != 0:
            self.status.zero_()
            raise KernelLibraryError(f"a kernel gave up waiting (code {code}); its results are invalid")

    # ---- embedding and norms --------------------------------------------------------------------
    def embed(self, token_ids, positions, tok_emb, pos_table, source=None, previous=None):
        """Rows of the embedding (plus rows of the position table).  With ``source``: a row whose
        source is >= 0 takes its id from ``previous[source]`` instead of ``token_ids``."""
        self._want(token_ids, torch.int32, "token_ids", 1)
        self._want(positions, torch.int32, "positions", 1)
        if source is not None:
            self._want(source, torch.int32, "token sources", 1)
            self._want(previous, torch.int32, "previous ids", 1)
            if source.numel() != token_ids.numel():
                raise KernelLibraryError("embed: one source per token")
        self._want(tok_emb, None, "tok_emb", 2)
        if pos_table is not None:
            self._want(pos_table, tok_emb.dtype, "pos_table", 2)
            if pos_table.shape[1] != tok_emb.shape[1]:
                raise KernelLibraryError("embed: position table and embedding differ in width")
        n, width = token_ids.numel(), tok_emb.shape[1]
        out = torch.empty((n, width), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_embed(_ptr(token_ids), _ptr(positions), _ptr(tok_emb), _ptr(pos_table),
                                _ptr(out), n, width, self._is_bf16(tok_emb), _ptr(source), _ptr(previous),
                                tok_emb.shape[0], pos_table.shape[0] if pos_table is not None else 0,
                                previous.numel() if previous is not None else 0, self._stream()),
              "embed")
        return out

    def layernorm(self, x32, gain, shift, eps, out_dtype):
        self._want(x32, torch.float32, "layernorm input", 2)
        self._want(gain, torch.float32, "layernorm gain", 1)
        if shift is not None:
            self._want(shift, torch.float32, "layernorm shift", 1)
        rows, width = x32.shape
        if gain.numel() != width:
            raise KernelLibraryError("layernorm: gain does not match the width")
        out = torch.empty((rows, width), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_layernorm(_ptr(x32), _ptr(gain), _ptr(shift), _ptr(out), rows, width,
                                    float(eps), self._is_bf16(out), self._stream()), "layernorm")
        return out

    def gather_rows(self, x32, rows):
        self._want(x32, torch.float32, "gather input", 2)
        self._want(rows, torch.int32, "rows", 1)
        out = torch.empty((rows.numel(), x32.shape[1]), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_gather_rows(_ptr(x32), _ptr(rows), _ptr(out), rows.numel(), x32.shape[1],
                                      x32.shape[0], self._stream()), "gather_rows")
        return out

    def gather_tokens(self, token_ids, source, previous):
        """token_ids[i] = previous[source[i]] for rows with source[i] >= 0 (in place): the tokens a
        step sampled become the next step's inputs without passing through the host."""
        for name, t in (("token_ids", token_ids), ("source", source), ("previous", previous)):
            self._want(t, torch.int32, name, 1)
        self._run(self.lib.mg_gather_tokens(_ptr(token_ids), _ptr(source), _ptr(previous),
                                            token_ids.numel(), previous.numel(), self._stream()), "gather_tokens")

    def upload_ints(self, dst, pinned) -> None:
        """dst[:] = pinned[:] where ``pinned`` is page-locked host memory: the device reads it
        itself, so nothing switches engines between this and the kernels that follow."""
        self._want(dst, torch.int32, "upload destination", 1)
        if (pinned.dtype != torch.int32 or pinned.device.type != "cpu" or not pinned.is_pinned()
                or pinned.numel() != dst.numel() or not pinned.is_contiguous()):
            raise KernelLibraryError("upload_ints: the source must be pinned int32 host memory of the same size")
        self._run(self.lib.mg_copy_ints(_ptr(dst), _ptr(pinned), dst.numel(), self._stream()), "upload_ints")

    # ---- projections ----------------------------------------------------------------------------
    def defer_layernorm(self, x32, gain, shift, eps, out_dtype, rows=None):
        """A LayerNorm to be fused into the projection that consumes it, where that pays."""
        self._want(x32, torch.float32, "layernorm input", 2)
        return DeferredNorm(self, x32, gain, shift, eps, out_dtype, rows)

    def _skinny_ok(self, m, k, dtype) -> bool:
        return (self.use_skinny and dtype == torch.bfloat16 and 0 < m <= SKINNY_ROWS and k % 8 == 0
                and SKINNY_ROWS * (2 * k + 64) + 8 * SKINNY_ROWS * 8 * 4 + 8 * k <= 200 * 1024)

    @staticmethod
    def _sink_args(kv_sink):
        """The key/value sink of a QKV projection as the C functions take it."""
        if kv_sink is None:
            return [None, None, None, 0, 0, 0, 0, 0]
        cache, slots, n_head, n_kv_head, head_dim = kv_sink
        return [_ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(slots), n_head * head_dim, n_kv_head,
                head_dim, cache.page_tokens, cache.k_pages.shape[0]]

    def _linear(self, x, weight, bias, epilogue, out, residual, kv_sink=None, greedy=None):
        """x: a tensor [M, K] or a DeferredNorm.  kv_sink: (cache view, slots, n_head, n_kv_head,
        head_dim) to also write key/value features to the cache.  greedy: (ids out, vocabulary
        limit) to also leave each row's argmax where the kernel that runs can take it on its way
        (``self.greedy_taken`` says whether it did).  Returns True if the sink was served inside
        the projection kernel."""
        deferred = x if isinstance(x, DeferredNorm) else None
        m, k = x.shape
        n = weight.shape[0]
        self._want(weight, None, "linear weight", 2)
        # which matrix followed which the last time: what a streaming kernel asks into L2 on its way
        if self._last_weight is not None:
            self._next_weight[self._last_weight] = weakref.ref(weight)
        self._last_weight = weight.data_ptr()
        if bias is not None:
            self._want(bias, torch.float32, "linear bias", 1)
        if weight.shape[1] != k or (bias is not None and bias.numel() != n):
            raise KernelLibraryError(
                f"linear: shapes do not fit: x {tuple(x.shape)}, w {tuple(weight.shape)}")
        out_bf16 = self._is_bf16(out) if out is not None else 0
        large = n >= STREAM_MIN_ROWS or (self.stream_min_bytes is not None and 2 * n * k >= self.stream_min_bytes)
        if self.use_wide and weight.dtype == torch.bfloat16 and 0 < m <= SKINNY_ROWS and k % 8 == 0 and large:
            # a matrix of many megabytes: whole rows as TMA boxes through a ring of stages, the first of
            # them asked for before the dependency wait
            if deferred is not None:
                args = [None, _ptr(deferred.x32), _ptr(deferred.rows), _ptr(deferred.gain),
                        _ptr(deferred.shift), deferred.eps]
            else:
                self._want(x, weight.dtype, "linear input", 2)
                args = [_ptr(x), None, None, None, None, 0.0]
            amax, parts = [None, None, 0], 0
            if greedy is not None:
                ids_out, limit = greedy
                parts = self.lib.mg_linear_wide_parts(m, n, k, 1 if deferred is not None else 0)
                part_v = torch.empty((m * parts,), dtype=torch.float32, device=self.device)
                part_i = torch.empty((m * parts,), dtype=torch.int32, device=self.device)
                amax = [_ptr(part_v), _ptr(part_i), int(limit or 0)]
            follower = self._next_weight.get(weight.data_ptr())
            follower = follower() if follower is not None and self.use_weight_prefetch else None
            ahead = [None, 0]
            if follower is not None and follower.is_cuda and follower.data_ptr() % 128 == 0:
                ahead = [_ptr(follower), min(follower.numel() * follower.element_size(), PREFETCH_MAX_BYTES) // 128]
            code = self.lib.mg_linear_wide(*args, _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                           m, n, k, epilogue, out_bf16, *self._sink_args(kv_sink), *amax,
                                           *ahead, _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (large matrix)")
                if greedy is not None:
                    self._run(self.lib.mg_argmax_merge(_ptr(part_v), _ptr(part_i), _ptr(ids_out), m, parts,
                                                       self._stream()), "argmax (merge)")
                    self.greedy_taken = True
                return kv_sink is not None
        if (self.use_stream and weight.dtype == torch.bfloat16 and 0 < m <= STREAM_ROWS and k % 8 == 0 and large):
            # a tall matrix (the head) or one of many megabytes: one CTA per SM streams it through
            # shared memory
            if deferred is not None and m > SKINNY_ROWS:
                # more rows than a CTA normalises quickly: the norm runs as a kernel of its own
                x, deferred = deferred.materialize(), None
            if deferred is not None:
                args = [None, _ptr(deferred.x32), _ptr(deferred.rows), _ptr(deferred.gain),
                        _ptr(deferred.shift), deferred.eps]
            else:
                self._want(x, weight.dtype, "linear input", 2)
                args = [_ptr(x), None, None, None, None, 0.0]
            amax = [None, None, 0]
            if greedy is not None:
                ids_out, limit = greedy
                parts = self.lib.mg_linear_stream_parts(n)
                part_v = torch.empty((m * parts,), dtype=torch.float32, device=self.device)
                part_i = torch.empty((m * parts,), dtype=torch.int32, device=self.device)
                amax = [_ptr(part_v), _ptr(part_i), int(limit or 0)]
            code = self.lib.mg_linear_stream(*args, _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                             m, n, k, epilogue, out_bf16, *self._sink_args(kv_sink), *amax,
                                             self.stream_max_chunks, _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (wide matrix)")
                if greedy is not None:
                    self._run(self.lib.mg_argmax_merge(_ptr(part_v), _ptr(part_i), _ptr(ids_out), m, parts,
                                                       self._stream()), "argmax (merge)")
                    self.greedy_taken = True
                return kv_sink is not None
        if self._skinny_ok(m, k, weight.dtype):
            sink = self._sink_args(kv_sink)
            if deferred is not None:
                args = [None, _ptr(deferred.x32), _ptr(deferred.rows), _ptr(deferred.gain),
                        _ptr(deferred.shift), deferred.eps]
            else:
                self._want(x, weight.dtype, "linear input", 2)
                args = [_ptr(x), None, None, None, None, 0.0]
            amax = [None, None, 0]
            if greedy is not None:
                # first stage of the argmax over the rows, on the projection's way
                ids_out, limit = greedy
                parts = self.lib.mg_linear_skinny_ctas(n, k)
                part_v = torch.empty((m * parts,), dtype=torch.float32, device=self.device)
                part_i = torch.empty((m * parts,), dtype=torch.int32, device=self.device)
                amax = [_ptr(part_v), _ptr(part_i), int(limit or 0)]
            code = self.lib.mg_linear_skinny(*args, _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                             m, n, k, epilogue, out_bf16, *sink, *amax, self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (small batch)")
                if greedy is not None:
                    self._run(self.lib.mg_argmax_merge(_ptr(part_v), _ptr(part_i), _ptr(ids_out), m, parts,
                                                       self._stream()), "argmax (merge)")
                    self.greedy_taken = True
                return kv_sink is not None
        if deferred is not None:
            x = deferred.materialize()
        self._want(x, weight.dtype, "linear input", 2)
        # (a matrix of thousands of 8-row tiles, the head, is left to the tensor-core GEMM: every one
        # of its clusters would stage the activations and meet at a barrier for a few KB of weights)
        # (and beyond 64 tokens it keeps only matrices of up to 3 MB: measured with 96 and 128 tokens, it
        # is faster than the tensor-core GEMM at 512 x 2048, slower from 3 x 768 x 768 elements on)
        if (x.dtype == torch.bfloat16 and self.use_cluster and 0 < m <= CLUSTER_ROWS and k % 8 == 0
                and n <= 8192 and (m <= 64 or 2 * n * k <= CLUSTER_WIDE_MAX_BYTES)):
            sink = self._sink_args(kv_sink)
            code = self.lib.mg_linear_cluster(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                              m, n, k, epilogue, out_bf16, *sink, self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (mid batch)")
                return kv_sink is not None
        if x.dtype == torch.bfloat16 and self.use_tensor_cores:
            # the key/value copy moves 16 bytes at a time: head sizes that are multiples of 8
            fused = kv_sink is not None and kv_sink[4] % 8 == 0
            sink = self._sink_args(kv_sink if fused else None)
            code = self.lib.mg_linear_tc(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                         m, n, k, epilogue, out_bf16, *sink, _ptr(self.status),
                                         self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (tensor cores)")
                return fused
        self._run(self.lib.mg_linear_simt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                      m, n, k, epilogue, self._is_bf16(x), out_bf16, self._stream()),
              "linear")
        return False

    def linear(self, x, weight, bias, activation, out_dtype):
        if activation not in ("none", "gelu_tanh"):
            raise KernelLibraryError(f"linear: no epilogue for activation {activation!r}")
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=self.device)
        self._linear(x, weight, bias, EPILOGUES[activation], out, None)
        return out

    def linear_qkv(self, x, weight, bias, n_head, n_kv_head, head_dim, cache, slots, out_dtype):
        """The fused q/k/v projection; new keys and values also go to their cache rows (inside
        the projection kernel where it can, else with the page-write kernel)."""
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=self.device)
        sink = None
        if cache is not None and cache.writes:
            self._want(slots, torch.int32, "slot_mapping", 1)
            sink = (cache, slots, n_head, n_kv_head, head_dim)
        stored = self._linear(x, weight, bias, EPILOGUES["none"], out, None, kv_sink=sink)
        if sink is not None and not stored:
            self.kv_store(out, n_head, n_kv_head, head_dim, cache, slots)
        return out

    def linear_residual(self, x, weight, bias, residual32):
        self._want(residual32, torch.float32, "residual", 2)
        if residual32.shape != (x.shape[0], weight.shape[0]):
            raise KernelLibraryError("linear_residual: residual has the wrong shape")
        self._linear(x, weight, bias, EPILOGUES["residual"], None, residual32)

    # ---- the whole feed-forward in one kernel (small batches) ---------------------------------------
    FUSED_MLP_ROWS = 16

    def _residual_ring(self, residual32):
        """Two more buffers like ``residual32`` that take turns with it as the residual stream
        (see ``mlp_residual``): ``(next, spare)``, ``next`` all zeros.  They are remembered by the
        tensor that currently holds the stream, so a chain of calls in one step allocates and
        zeroes once."""
        entry = self._ring
        if entry is not None and entry[0] is residual32:
            return entry[1], entry[2]
        nxt = torch.empty_like(residual32)
        spare = torch.empty_like(residual32)
        self._run(self.lib.mg_zero_fill(_ptr(nxt), nxt.numel() * 4, self._stream()), "zero fill")
        return nxt, spare

    def _packed_proj(self, weight):
        """The second matrix of a feed-forward, [C, F], copied once into the order in which the
        fused kernel's lanes read it (``mg_mlp_pack_elements`` in mlp_fused.cu): a layout change
        made when a matrix is first seen, not a computation of the step."""
        key = weight.data_ptr()
        hit = self._packed.get(key)
        if hit is not None and hit[0] is weight:
            return hit[1]
        c, f = weight.shape
        groups = (f + 15) // 16
        padded = weight
        if groups * 16 != f:
            padded = torch.zeros((c, groups * 16), dtype=weight.dtype, device=weight.device)
            padded[:, :f] = weight
        packed = padded.view(c // 8, 8, groups, 4, 4).permute(2, 0, 1, 3, 4).contiguous()
        assert packed.numel() == self.lib.mg_mlp_pack_elements(c, f)
        self._packed[key] = (weight, packed)
        return packed

    def mlp_residual(self, y, fc_weight, fc_bias, proj_weight, proj_bias, activation, residual32, act_dtype):
        """``residual32 + proj(act(fc(y)))``.  Returns the tensor that holds the sum: ``residual32``
        itself (added in place by two projection kernels), or, where the whole feed-forward runs as
        one kernel (bfloat16, up to 16 tokens, ``y`` a deferred LayerNorm of ``residual32``),
        another tensor: that kernel cannot write where its CTAs still read, so the residual
        stream moves between three buffers that take turns."""
        deferred = y if isinstance(y, DeferredNorm) else None
        m = residual32.shape[0]
        if (self.use_fused_mlp and deferred is not None and deferred.rows is None and deferred.x32 is residual32
                and activation == "gelu_tanh" and fc_weight.dtype == torch.bfloat16 and act_dtype == torch.bfloat16
                and deferred.dtype == torch.bfloat16 and 0 < m <= self.FUSED_MLP_ROWS
                and residual32.shape[1] <= self.lib.mg_mlp_fused_max_width() and residual32.shape[1] % 8 == 0
                and fc_weight.shape[0] % 8 == 0):
            self._want(residual32, torch.float32, "residual", 2)
            self._want(fc_weight, torch.bfloat16, "fc weight", 2)
            self._want(proj_weight, torch.bfloat16, "proj weight", 2)
            c, f = residual32.shape[1], fc_weight.shape[0]
            if fc_weight.shape != (f, c) or proj_weight.shape != (c, f):
                raise KernelLibraryError("feed-forward: the two matrices do not fit the width")
            for b, n, name in ((fc_bias, f, "fc bias"), (proj_bias, c, "proj bias")):
                if b is not None and self._want(b, torch.float32, name, 1).numel() != n:
                    raise KernelLibraryError(f"feed-forward: {name} has the wrong length")
            nxt, spare = self._residual_ring(residual32)
            code = self.lib.mg_mlp_fused(_ptr(residual32), _ptr(nxt), _ptr(spare), _ptr(deferred.gain),
                                         _ptr(deferred.shift), deferred.eps, _ptr(fc_weight), _ptr(fc_bias),
                                         _ptr(self._packed_proj(proj_weight)), _ptr(proj_bias), m, c, f,
                                         self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "feed-forward (fused)")
                self._ring = (nxt, spare, residual32)          # nxt holds the stream; spare is zero
                return nxt
            self._ring = None
        h = self.linear(y, fc_weight, fc_bias, activation, act_dtype)
        self.linear_residual(h, proj_weight, proj_bias, residual32)
        return residual32

    def logits(self, y, tok_emb, greedy_out=None, vocab_limit=None):
        """Logits in 32-bit.  With ``greedy_out`` (int32 ``[rows]``): the argmax of every row (ids at
        or above ``vocab_limit`` excluded) is left there as well; returns ``(logits, taken)`` then,
        ``taken`` False if the projection that ran cannot take it on its way."""
        if greedy_out is None:
            return self.linear(y, tok_emb, None, "none", torch.float32)
        self._ids_out(greedy_out, y.shape[0])
        out = torch.empty((y.shape[0], tok_emb.shape[0]), dtype=torch.float32, device=self.device)
        self.greedy_taken = False
        self._linear(y, tok_emb, None, EPILOGUES["none"], out, None, greedy=(greedy_out, vocab_limit))
        return out, self.greedy_taken

    # ---- attention ------------------------------------------------------------------------------
    def kv_store(self, qkv, n_head, n_kv_head, head_dim, cache, slot_mapping):
        self._want(qkv, cache.k_pages.dtype, "qkv", 2)
        self._want(slot_mapping, torch.int32, "slot_mapping", 1)
        self._want(cache.k_pages, None, "k_pages", 4)
        self._want(cache.v_pages, cache.k_pages.dtype, "v_pages", 4)
        if qkv.shape[1] != (n_head + 2 * n_kv_head) * head_dim:
            raise KernelLibraryError("kv_store: qkv width does not match the head sizes")
        if tuple(cache.k_pages.shape[1:]) != (n_kv_head, cache.page_tokens, head_dim):
            raise KernelLibraryError("kv_store: page storage does not match the head sizes")
        self._run(self.lib.mg_kv_store(_ptr(qkv), _ptr(slot_mapping), _ptr(cache.k_pages),
                                   _ptr(cache.v_pages), qkv.shape[0], n_head, n_kv_head, head_dim,
                                   cache.page_tokens, cache.k_pages.shape[0], self._is_bf16(qkv),
                                   self._stream()), "kv_store")

    SPLIT_HEAD_DIMS = (16, 32, 64, 128, 256)

    PREFILL_TC_HEAD_DIMS = (64,)

    def _attention_tiles_name(self, n_head: int) -> str:
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # work items of the tiled kernel that run at once, per head (two CTAs per SM)
        return f"attention_tiles/{max(1, 2 * self._sm_count // n_head)}"

    def plan_prompt_attention(self, batch, plan, n_head, n_kv_head, head_dim) -> None:
        """Host half of the tiled prompt attention: the work list of a step (``attention_plan``),
        added to ``plan`` under a name that layers of equal head count share.  Nothing is planned
        for steps that the tiled kernel does not serve."""
        if (batch.decode_only or batch.act_dtype != torch.bfloat16 or not self.use_tensor_cores
                or not self.use_prefill_tc or head_dim not in self.PREFILL_TC_HEAD_DIMS):
            return
        name = self._attention_tiles_name(n_head)
        if name not in plan.arrays:
            import numpy as np

            slots = int(name.rsplit("/", 1)[1])
            # (steps of a shape that came before take their list from a small table)
            key = (tuple(batch.q_len), tuple(batch.ctx_before), slots)
            work = self._tile_lists.get(key)
            if work is None:
                work = np.asarray(query_tiles(batch.q_len, batch.ctx_before, slots), dtype=np.int32).reshape(-1, 5)
                if len(self._tile_lists) >= 64:
                    self._tile_lists.pop(next(iter(self._tile_lists)))
                self._tile_lists[key] = work
            plan.arrays[name] = work.copy()                  # (the table's copy stays as it is)
            plan.signature.append(("attention_merge", batch.max_ctx_after > KEY_CHUNK))

    def paged_attention(self, qkv, n_head, n_kv_head, head_dim, scale, cache, ctx):
        self._want(qkv, cache.k_pages.dtype, "qkv", 2)
        table = self._want(ctx.block_tables[cache.group], torch.int32, "block_table", 2)
        n = qkv.shape[0]
        out = torch.empty((n, n_head * head_dim), dtype=qkv.dtype, device=self.device)
        window = int(cache.window or 0)
        if (qkv.dtype == torch.bfloat16 and getattr(ctx, "decode_only", False)
                and head_dim in self.SPLIT_HEAD_DIMS and self.use_split_attention):
            # single query tokens: split along the keys; the last block of each row merges
            splits = self.lib.mg_attention_split_count(int(ctx.max_ctx_after), window, head_dim)
            floats = self.lib.mg_attention_split_scratch_floats(n, n_head, head_dim, splits)
            scratch = torch.empty((floats,), dtype=torch.float32, device=self.device)
            self._run(self.lib.mg_paged_attention_split(
                _ptr(qkv), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(table),
                _ptr(ctx.token_request), _ptr(ctx.positions), _ptr(out), _ptr(scratch),
                _ptr(self._counters(n * n_head)), n, n_head, n_kv_head, head_dim, cache.page_tokens,
                table.shape[1], window, splits, float(scale), cache.k_pages.shape[0], table.shape[0],
                _ptr(self.status), self._stream()),
                "paged_attention (split)")
            # a grid of several waves merges in a kernel of its own
            self.launches += self.lib.mg_attention_split_launches(n, n_head, n_kv_head, splits) - 1
            return out
        work = getattr(ctx, "extra", {}).get(self._attention_tiles_name(n_head))
        if (qkv.dtype == torch.bfloat16 and work is not None and work.shape[0] > 0
                and self.use_tensor_cores and self.use_prefill_tc
                and head_dim in self.PREFILL_TC_HEAD_DIMS):
            # portions of prompts: query tiles of 128 on the tensor cores
            self._want(work, torch.int32, "attention tiles", 2)
            # tiles cut along the keys leave partial rows in scratch; the part that finishes last merges them
            merge = int(ctx.max_ctx_after > KEY_CHUNK)
            partial = counters = None
            if merge:
                floats = self.lib.mg_attention_prefill_scratch_floats(work.shape[0], n_head)
                partial = torch.empty((floats,), dtype=torch.float32, device=self.device)
                counters = self._counters(work.shape[0] * n_head)
            code = self.lib.mg_attention_prefill_tc(
                _ptr(qkv), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(work), _ptr(table),
                _ptr(ctx.positions), _ptr(out), _ptr(partial), _ptr(counters), merge, work.shape[0], n, n_head,
                n_kv_head, head_dim,
                cache.page_tokens, cache.k_pages.shape[0], table.shape[1], window, float(scale),
                table.shape[0], _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "paged_attention (prefill, tensor cores)")
                return out
        self._run(self.lib.mg_paged_attention_generic(
            _ptr(qkv), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(table),
            _ptr(ctx.token_request), _ptr(ctx.positions), _ptr(out), n, n_head, n_kv_head, head_dim,
            cache.page_tokens, table.shape[1], window, float(scale), cache.k_pages.shape[0], table.shape[0],
            self._is_bf16(qkv), self._stream()), "paged_attention")
        return out

    # ---- sampling -------------------------------------------------------------------------------
    def _ids_out(self, out, rows):
        if out is None:
            return torch.empty((rows,), dtype=torch.int32, device=self.device)
        self._want(out, torch.int32, "ids", 1)
        if out.numel() != rows:
            raise KernelLibraryError(f"ids: room for {out.numel()} rows, {rows} wanted")
        return out

    def argmax(self, logits, vocab_limit=None, out=None):
        self._want(logits, torch.float32, "logits", 2)
        rows, vocab = logits.shape
        out = self._ids_out(out, rows)
        if vocab >= 8192 and rows <= 512:
            # few rows of a wide vocabulary: many blocks per row, then a merge
            parts = self.lib.mg_argmax_parts(vocab)
            scratch_v = torch.empty((rows * parts,), dtype=torch.float32, device=self.device)
            scratch_i = torch.empty((rows * parts,), dtype=torch.int32, device=self.device)
            self._run(self.lib.mg_argmax_wide(_ptr(logits), _ptr(out), _ptr(scratch_v),
                                          _ptr(scratch_i), rows, vocab, int(vocab_limit or 0),
                                          self._stream()), "argmax (wide)")
            self.launches += 1
            return out
        self._run(self.lib.mg_argmax(_ptr(logits), _ptr(out), rows, vocab,
                                 int(vocab_limit or 0), self._stream()), "argmax")
        return out

    def sample(self, logits, temperature, top_k, top_p, seed_lo, seed_hi, counter, vocab_limit=None,
               out=None):
        """One draw per row.  temperature float32 [rows]; top_k int32 [rows] or None (<= 0: off);
        top_p float32 [rows] or None (>= 1: off); seed_lo, seed_hi, counter: int32 [rows] holding
        the 32-bit words of each row's seed and the number of its draw."""
        self._want(logits, torch.float32, "logits", 2)
        rows = logits.shape[0]
        self._want(temperature, torch.float32, "temperature", 1)
        for name, t in (("top_k", top_k), ("seed_lo", seed_lo), ("seed_hi", seed_hi),
                        ("counter", counter)):
            if t is not None:
                self._want(t, torch.int32, name, 1)
        if top_p is not None:
            self._want(top_p, torch.float32, "top_p", 1)
        for t in (temperature, top_k, top_p, seed_lo, seed_hi, counter):
            if t is not None and t.numel() != rows:
                raise KernelLibraryError("sample: per-row parameters do not match the rows")
        out = self._ids_out(out, rows)
        self._run(self.lib.mg_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                 _ptr(seed_lo), _ptr(seed_hi), _ptr(counter), _ptr(out), rows,
                                 logits.shape[1], int(vocab_limit or 0), self._stream()), "sample")
        return out


_default = {}


def default_ops(device="cuda:0") -> CudaOps:
    key = str(torch.device(device))
    if key not in _default:
        _default[key] = CudaOps(device)
    return _default[key]
