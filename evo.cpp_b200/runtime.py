"""ctypes binding of the evo_* model/context C ABI (include/evo/evo.h).

The same binding drives this repository's libevo.so and, in tests and the
CPU-baseline legs of the benchmark, upstream's own CPU build of the same ABI
(oracle/_ref/libevo_ref.so) - the two are interchangeable behind it.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

BACKEND_AUTO, BACKEND_CUDA, BACKEND_CPU = 0, 1, 2
MODEL_FLAG_ALLOW_SYNTHETIC = 1
CONTEXT_FLAG_FAST_Q8_KV = 1 << 0
CONTEXT_FLAG_TENSORCORE_FP8 = 1 << 8
CONTEXT_FLAG_FULL_ARENA = 1 << 9
CONTEXT_FLAG_FP8_FFN = 1 << 10

DUMP_POINTS = ("block_output", "pre_norm", "mixer_input_projection", "mixer_short_filter", "mixer_short_state",
               "mixer_inner_state", "mixer_x2", "mixer_x1", "mixer_value", "mixer_pregate", "mixer_state",
               "mixer_filter", "mixer_convolution", "mixer_output", "mixer_projection", "mixer_residual",
               "post_norm", "mlp_l1", "mlp_l2", "mlp_activation", "mlp_gated", "mlp_output")

DUMP_CALLBACK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_size_t, ctypes.c_int32, ctypes.POINTER(ctypes.c_float),
                                 ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p)

LOGITS_CALLBACK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t,
                                   ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p)


class DumpRequest(ctypes.Structure):
    _fields_ = [("layer", ctypes.c_size_t), ("point", ctypes.c_int32)]


class ModelParams(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("backend", ctypes.c_int),
                ("devices", ctypes.POINTER(ctypes.c_int32)), ("device_count", ctypes.c_size_t),
                ("flags", ctypes.c_uint32)]


class ModelConfig(ctypes.Structure):
    """evo_b200_model_config (include/evo/evo_b200.h)."""
    _fields_ = ([("struct_size", ctypes.c_size_t), ("model_id", ctypes.c_char * 64), ("architecture", ctypes.c_char * 64),
                 ("artifact_profile", ctypes.c_char * 64)] +
                [(name, ctypes.c_size_t) for name in
                 ("vocab_size", "width", "layers", "heads", "state_size", "inner_width", "short_filter_length",
                  "hcs_filter_length", "hcm_filter_length", "hcs_filter_groups", "hcm_filter_groups", "max_seqlen")] +
                [(name, ctypes.c_float) for name in ("epsilon", "rope_scale", "rope_base")] +
                [(name, ctypes.c_int32) for name in
                 ("qkv_source_head_major", "hyena_projection_e4m3", "hcm_filter_f32", "test_fixture")])


class ContextParams(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("context_size", ctypes.c_size_t),
                ("flags", ctypes.c_uint32)]


class SamplerParams(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("temperature", ctypes.c_float),
                ("top_k", ctypes.c_size_t), ("top_p", ctypes.c_float), ("seed", ctypes.c_uint64)]


class StageInfo(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("device", ctypes.c_int32),
                ("layer_begin", ctypes.c_size_t), ("layer_end", ctypes.c_size_t),
                ("weight_bytes", ctypes.c_size_t), ("cache_bytes", ctypes.c_size_t),
                ("arena_bytes", ctypes.c_size_t)]


class SchedulerParams(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("workers", ctypes.c_size_t), ("maximum_queue", ctypes.c_size_t),
                ("context_size", ctypes.c_size_t), ("context_flags", ctypes.c_uint32)]


class Request(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("kind", ctypes.c_int32), ("sequence", ctypes.c_char_p),
                ("length", ctypes.c_size_t), ("new_tokens", ctypes.c_size_t), ("sampler", SamplerParams)]


class RequestResult(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("status", ctypes.c_int), ("error", ctypes.c_char_p),
                ("cancelled", ctypes.c_int32), ("log_likelihood", ctypes.c_double), ("scored_tokens", ctypes.c_size_t),
                ("token_log_likelihoods", ctypes.POINTER(ctypes.c_double)),
                ("generated", ctypes.POINTER(ctypes.c_uint8)), ("generated_length", ctypes.c_size_t),
                ("queue_seconds", ctypes.c_double), ("run_seconds", ctypes.c_double)]


class SchedulerMetrics(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t)] + [(n, ctypes.c_uint64) for n in
                ("submitted", "rejected", "completed", "failed", "cancelled")] + [
                (n, ctypes.c_size_t) for n in ("queued", "queue_peak", "active", "active_peak")]


REQUEST_CALLBACK = ctypes.CFUNCTYPE(None, ctypes.c_uint64, ctypes.POINTER(RequestResult), ctypes.c_void_p)


class EvoError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


class EvoLibrary:
    def __init__(self, path: Path):
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(f"{path} is missing (build it first; there is no fallback)")
        lib = self.lib = ctypes.CDLL(str(path))
        V, Z, I = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        lib.evo_last_error.restype = ctypes.c_char_p
        lib.evo_version_string.restype = ctypes.c_char_p
        lib.evo_abi_version.restype = ctypes.c_uint32
        lib.evo_model_default_params.restype = ModelParams
        lib.evo_context_default_params.restype = ContextParams
        lib.evo_sampler_default_params.restype = SamplerParams
        lib.evo_model_load.argtypes = [ctypes.c_char_p, ctypes.POINTER(ModelParams), ctypes.POINTER(V)]
        lib.evo_model_free.argtypes = [V]
        for name in ("evo_model_id", "evo_model_architecture", "evo_model_profile"):
            getattr(lib, name).restype = ctypes.c_char_p
            getattr(lib, name).argtypes = [V]
        for name in ("evo_model_vocab_size", "evo_model_max_context", "evo_model_embedding_width",
                     "evo_model_layer_count"):
            getattr(lib, name).restype = Z
            getattr(lib, name).argtypes = [V]
        lib.evo_context_create.argtypes = [V, ctypes.POINTER(ContextParams), ctypes.POINTER(V)]
        lib.evo_context_free.argtypes = [V]
        lib.evo_context_position.restype = Z
        lib.evo_context_position.argtypes = [V]
        lib.evo_context_capacity.restype = Z
        lib.evo_context_capacity.argtypes = [V]
        lib.evo_context_profile.restype = ctypes.c_char_p
        lib.evo_context_profile.argtypes = [V]
        lib.evo_context_prefill.argtypes = [V, V, LOGITS_CALLBACK, V]
        lib.evo_context_decode.argtypes = [V, ctypes.c_uint32, LOGITS_CALLBACK, V]
        lib.evo_context_embed.argtypes = [V, V, Z, LOGITS_CALLBACK, V]
        lib.evo_batch_create.argtypes = [Z, ctypes.POINTER(V)]
        lib.evo_batch_free.argtypes = [V]
        lib.evo_batch_clear.argtypes = [V]
        lib.evo_batch_add_sequence.argtypes = [V, ctypes.c_char_p, Z]
        lib.evo_sampler_create.argtypes = [ctypes.POINTER(SamplerParams), ctypes.POINTER(V)]
        lib.evo_sampler_free.argtypes = [V]
        lib.evo_sampler_sample.argtypes = [V, ctypes.POINTER(ctypes.c_float), Z,
                                           ctypes.POINTER(ctypes.c_uint32)]
        self.has_extensions = hasattr(lib, "evo_b200_context_prefill_device")
        if self.has_extensions:
            lib.evo_b200_context_prefill_device.argtypes = [V, V, Z, I, ctypes.POINTER(V)]
            lib.evo_b200_context_continue_device.argtypes = [V, V, Z, ctypes.POINTER(V)]
            lib.evo_b200_context_prefill_tokens.argtypes = [V, ctypes.POINTER(ctypes.c_uint32), Z, ctypes.c_int32,
                                                            LOGITS_CALLBACK, V]
            lib.evo_b200_context_embed_tokens.argtypes = [V, ctypes.POINTER(ctypes.c_uint32), Z, Z, ctypes.c_int32,
                                                          LOGITS_CALLBACK, V]
            lib.evo_b200_context_activation_capacity.restype = Z
            lib.evo_b200_context_activation_capacity.argtypes = [V]
            lib.evo_b200_read_model_config.argtypes = [ctypes.c_char_p, ctypes.c_int32, ctypes.POINTER(ModelConfig),
                                                       ctypes.POINTER(ctypes.c_uint8), Z]
            lib.evo_b200_context_stream.restype = V
            lib.evo_b200_context_stream.argtypes = [V]
            lib.evo_b200_context_synchronize.argtypes = [V]
            lib.evo_b200_context_stage_count.restype = Z
            lib.evo_b200_context_stage_count.argtypes = [V]
            lib.evo_b200_context_stage_info.argtypes = [V, Z, ctypes.POINTER(StageInfo)]
            lib.evo_b200_context_profile_enable.argtypes = [V, I]
            lib.evo_b200_context_profile_read.restype = Z
            lib.evo_b200_context_profile_read.argtypes = [V, ctypes.POINTER(ctypes.c_double),
                                                          ctypes.POINTER(ctypes.c_uint64), Z]
            lib.evo_b200_profile_category_name.restype = ctypes.c_char_p
            lib.evo_b200_profile_category_name.argtypes = [Z]
            lib.evo_b200_dump_point_name.restype = ctypes.c_char_p
            lib.evo_b200_dump_point_name.argtypes = [ctypes.c_int32]
            lib.evo_b200_context_prefill_with_dumps.argtypes = [V, V, ctypes.POINTER(DumpRequest), Z, I,
                                                                DUMP_CALLBACK, LOGITS_CALLBACK, V]
            lib.evo_b200_context_decode_with_dumps.argtypes = [V, ctypes.c_uint32, ctypes.POINTER(DumpRequest), Z,
                                                               DUMP_CALLBACK, LOGITS_CALLBACK, V]
            lib.evo_b200_scheduler_create.argtypes = [V, ctypes.POINTER(SchedulerParams), ctypes.POINTER(V)]
            lib.evo_b200_scheduler_free.argtypes = [V]
            lib.evo_b200_scheduler_submit.argtypes = [V, ctypes.POINTER(Request), REQUEST_CALLBACK, V,
                                                      ctypes.POINTER(ctypes.c_uint64)]
            lib.evo_b200_scheduler_cancel.argtypes = [V, ctypes.c_uint64]
            lib.evo_b200_scheduler_read_metrics.argtypes = [V, ctypes.POINTER(SchedulerMetrics)]
            lib.evo_b200_scheduler_wait_idle.argtypes = [V]
            lib.evo_b200_model_load_slice.argtypes = [ctypes.c_char_p, ctypes.c_int32, Z, Z,
                                                      ctypes.c_uint32, ctypes.POINTER(V)]
            lib.evo_b200_context_slice_embed.argtypes = [V, V, Z, Z]
            lib.evo_b200_context_slice_run.argtypes = [V, Z, Z]
            lib.evo_b200_context_slice_head.argtypes = [V, Z, Z, ctypes.POINTER(V)]
            lib.evo_b200_context_slice_hidden.restype = V
            lib.evo_b200_context_slice_hidden.argtypes = [V]

    def read_model_config(self, path, allow_test_fixture: bool = False):
        """(ModelConfig, mixer codes per block: 0 HCS, 1 HCM, 2 HCL, 3 attention) without loading weights."""
        config = ModelConfig()
        config.struct_size = ctypes.sizeof(ModelConfig)
        mixers = (ctypes.c_uint8 * 4096)()
        self.check(self.lib.evo_b200_read_model_config(str(path).encode(), int(allow_test_fixture), ctypes.byref(config),
                                                       mixers, 4096))
        return config, list(mixers[:config.layers])

    def check(self, status: int) -> None:
        if status != 0:
            raise EvoError(status, (self.lib.evo_last_error() or b"").decode())

    def load(self, path, *, backend=BACKEND_AUTO, devices=None, flags=0) -> "Model":
        params = self.lib.evo_model_default_params()
        params.backend = backend
        params.flags = flags
        keep = None
        if devices:
            keep = (ctypes.c_int32 * len(devices))(*devices)
            params.devices = ctypes.cast(keep, ctypes.POINTER(ctypes.c_int32))
            params.device_count = len(devices)
        handle = ctypes.c_void_p()
        self.check(self.lib.evo_model_load(str(path).encode(), ctypes.byref(params), ctypes.byref(handle)))
        return Model(self, handle)

    def load_slice(self, path, device: int, slice_index: int, slice_count: int, flags=0) -> "Model":
        """Stage `slice_index` of a `slice_count`-process layer pipeline on `device`."""
        handle = ctypes.c_void_p()
        self.check(self.lib.evo_b200_model_load_slice(str(path).encode(), device, slice_index, slice_count,
                                                      flags, ctypes.byref(handle)))
        return Model(self, handle)


class Model:
    def __init__(self, library: EvoLibrary, handle):
        self.library, self.handle = library, handle

    def close(self) -> None:
        if self.handle:
            self.library.lib.evo_model_free(self.handle)
            self.handle = None

    @property
    def vocab(self) -> int:
        return self.library.lib.evo_model_vocab_size(self.handle)

    @property
    def width(self) -> int:
        return self.library.lib.evo_model_embedding_width(self.handle)

    @property
    def layers(self) -> int:
        return self.library.lib.evo_model_layer_count(self.handle)

    @property
    def model_id(self) -> str:
        return self.library.lib.evo_model_id(self.handle).decode()

    def context(self, context_size: int = 4096, flags: int = 0) -> "Context":
        params = self.library.lib.evo_context_default_params()
        params.context_size = context_size
        params.flags = flags
        handle = ctypes.c_void_p()
        self.library.check(self.library.lib.evo_context_create(self.handle, ctypes.byref(params),
                                                               ctypes.byref(handle)))
        return Context(self.library, handle, self.vocab, self.width)


class Scheduler:
    """Worker pool over shared-weight contexts of one model (evo_b200_scheduler_*).  Results are
    collected in `results[ticket]` as plain dicts by the completion callback."""

    def __init__(self, model: "Model", workers: int, maximum_queue: int, context_size: int, flags: int = 0):
        import threading

        self.library = model.library
        params = SchedulerParams(ctypes.sizeof(SchedulerParams), workers, maximum_queue, context_size, flags)
        self.handle = ctypes.c_void_p()
        self.library.check(self.library.lib.evo_b200_scheduler_create(model.handle, ctypes.byref(params),
                                                                      ctypes.byref(self.handle)))
        self.results: dict[int, dict] = {}
        self._lock = threading.Lock()

        @REQUEST_CALLBACK
        def on_done(ticket, result, _user):
            r = result.contents
            entry = {"status": r.status, "error": (r.error or b"").decode(), "cancelled": bool(r.cancelled),
                     "log_likelihood": r.log_likelihood, "scored_tokens": r.scored_tokens,
                     "token_log_likelihoods": [r.token_log_likelihoods[i] for i in range(r.scored_tokens)],
                     "generated": bytes(r.generated[i] for i in range(r.generated_length)),
                     "queue_seconds": r.queue_seconds, "run_seconds": r.run_seconds}
            with self._lock:
                self.results[ticket] = entry

        self._callback = on_done

    def _submit(self, kind: int, payload: bytes, new_tokens: int = 0, **sampler) -> int:
        request = Request()
        request.struct_size = ctypes.sizeof(Request)
        request.kind, request.sequence, request.length, request.new_tokens = kind, payload, len(payload), new_tokens
        request.sampler = self.library.lib.evo_sampler_default_params()
        for name, value in sampler.items():
            setattr(request.sampler, name, value)
        ticket = ctypes.c_uint64()
        self.library.check(self.library.lib.evo_b200_scheduler_submit(self.handle, ctypes.byref(request),
                                                                      self._callback, None, ctypes.byref(ticket)))
        return ticket.value

    def score(self, sequence: bytes) -> int:
        """Ticket of the queued request, 0 when the queue was full."""
        return self._submit(0, bytes(sequence))

    def generate(self, prompt: bytes, tokens: int, **sampler) -> int:
        return self._submit(1, bytes(prompt), tokens, **sampler)

    def cancel(self, ticket: int) -> bool:
        return bool(self.library.lib.evo_b200_scheduler_cancel(self.handle, ticket))

    def wait_idle(self) -> None:
        self.library.lib.evo_b200_scheduler_wait_idle(self.handle)

    def metrics(self) -> dict:
        m = SchedulerMetrics()
        m.struct_size = ctypes.sizeof(SchedulerMetrics)
        self.library.check(self.library.lib.evo_b200_scheduler_read_metrics(self.handle, ctypes.byref(m)))
        return {name: int(getattr(m, name)) for name, _ in SchedulerMetrics._fields_[1:]}

    def close(self) -> None:
        if self.handle:
            self.library.lib.evo_b200_scheduler_free(self.handle)
            self.handle = None


class Context:
    def __init__(self, library: EvoLibrary, handle, vocab: int, width: int):
        self.library, self.handle, self.vocab, self.width = library, handle, vocab, width

    def close(self) -> None:
        if self.handle:
            self.library.lib.evo_context_free(self.handle)
            self.handle = None

    @property
    def position(self) -> int:
        return self.library.lib.evo_context_position(self.handle)

    @property
    def profile(self) -> str:
        return self.library.lib.evo_context_profile(self.handle).decode()

    def _collect(self, call, columns: int) -> np.ndarray:
        chunks: list[tuple[int, np.ndarray]] = []

        @LOGITS_CALLBACK
        def on_rows(data, rows, cols, offset, _user):
            chunks.append((offset, np.ctypeslib.as_array(data, shape=(rows, cols)).copy()))
            return 0

        self.library.check(call(on_rows))
        chunks.sort(key=lambda c: c[0])
        return np.concatenate([c[1] for c in chunks], axis=0) if chunks else np.zeros((0, columns), np.float32)

    def _batch(self, sequence: bytes):
        lib = self.library.lib
        batch = ctypes.c_void_p()
        self.library.check(lib.evo_batch_create(1, ctypes.byref(batch)))
        try:
            self.library.check(lib.evo_batch_add_sequence(batch, sequence, len(sequence)))
        except Exception:
            lib.evo_batch_free(batch)
            raise
        return batch

    def prefill(self, sequence: bytes) -> np.ndarray:
        """Chunked prefill of raw bytes; returns F32 logits [tokens, vocab]."""
        batch = self._batch(bytes(sequence))
        try:
            return self._collect(lambda cb: self.library.lib.evo_context_prefill(self.handle, batch, cb, None),
                                 self.vocab)
        finally:
            self.library.lib.evo_batch_free(batch)

    PREFILL_FRESH, PREFILL_STATELESS, PREFILL_CACHED, PREFILL_CHUNK = 0, 1, 2, 3

    def prefill_tokens(self, tokens, mode: int = 0) -> np.ndarray:
        """evo_b200_context_prefill_tokens: token ids, one of the PREFILL_* forms; F32 logits [tokens, vocab]."""
        ids = (ctypes.c_uint32 * len(tokens))(*tokens)
        return self._collect(lambda cb: self.library.lib.evo_b200_context_prefill_tokens(
            self.handle, ids, len(tokens), mode, cb, None), self.vocab)

    def embed_tokens(self, tokens, layer: int, first_chunk: bool = True) -> np.ndarray:
        """evo_b200_context_embed_tokens: block output of `layer` for one chunk of token ids, F32 [tokens, width]."""
        ids = (ctypes.c_uint32 * len(tokens))(*tokens)
        return self._collect(lambda cb: self.library.lib.evo_b200_context_embed_tokens(
            self.handle, ids, len(tokens), layer, int(first_chunk), cb, None), self.width)

    @property
    def activation_capacity(self) -> int:
        return self.library.lib.evo_b200_context_activation_capacity(self.handle)

    def decode(self, token: int) -> np.ndarray:
        return self._collect(lambda cb: self.library.lib.evo_context_decode(self.handle, token, cb, None),
                             self.vocab)[0]

    def embed(self, sequence: bytes, layer: int) -> np.ndarray:
        batch = self._batch(bytes(sequence))
        try:
            return self._collect(lambda cb: self.library.lib.evo_context_embed(self.handle, batch, layer, cb, None),
                                 self.width)
        finally:
            self.library.lib.evo_batch_free(batch)

    # ---- extensions of this repository's library
    def _with_dumps(self, taps, call, consume=None):
        """taps: iterable of (layer, point name).  Returns (logits, {(layer, name): array}); with
        `consume` the arrays are handed to consume(layer, name, array) instead of being kept."""
        taps = list(taps)
        requests = (DumpRequest * max(1, len(taps)))()
        for slot, (layer, name) in zip(requests, taps):
            slot.layer, slot.point = layer, DUMP_POINTS.index(name)
        collected: dict = {}

        @DUMP_CALLBACK
        def on_dump(layer, point, data, rows, cols, _user):
            values = np.ctypeslib.as_array(data, shape=(rows, cols))
            if consume is not None:
                return int(consume(layer, DUMP_POINTS[point], values) or 0)
            collected[(layer, DUMP_POINTS[point])] = values.copy()
            return 0

        logits = self._collect(lambda cb: call(requests, len(taps), on_dump, cb), self.vocab)
        return logits, collected

    def prefill_with_dumps(self, sequence: bytes, taps, cached: bool = False, consume=None):
        batch = self._batch(bytes(sequence))
        try:
            return self._with_dumps(taps, lambda r, n, d, cb: self.library.lib.evo_b200_context_prefill_with_dumps(
                self.handle, batch, r, n, int(cached), d, cb, None), consume)
        finally:
            self.library.lib.evo_batch_free(batch)

    def decode_with_dumps(self, token: int, taps, consume=None):
        logits, dumps = self._with_dumps(taps, lambda r, n, d, cb: self.library.lib.evo_b200_context_decode_with_dumps(
            self.handle, token, r, n, d, cb, None), consume)
        return logits[0], dumps

    def prefill_device(self, device_tokens: int, rows: int, stateless: bool = True) -> int:
        out = ctypes.c_void_p()
        self.library.check(self.library.lib.evo_b200_context_prefill_device(
            self.handle, device_tokens, rows, int(stateless), ctypes.byref(out)))
        return out.value

    def continue_device(self, device_tokens: int, rows: int) -> int:
        out = ctypes.c_void_p()
        self.library.check(self.library.lib.evo_b200_context_continue_device(
            self.handle, device_tokens, rows, ctypes.byref(out)))
        return out.value

    def stream(self) -> int:
        return self.library.lib.evo_b200_context_stream(self.handle)

    def synchronize(self) -> None:
        self.library.check(self.library.lib.evo_b200_context_synchronize(self.handle))

    def profile_enable(self, enabled: bool = True) -> None:
        self.library.check(self.library.lib.evo_b200_context_profile_enable(self.handle, int(enabled)))

    def profile_read(self) -> dict[str, tuple[float, int]]:
        """{operator class: (milliseconds, launches)} since profiling was enabled."""
        lib = self.library.lib
        count = lib.evo_b200_context_profile_read(self.handle, None, None, 0)
        ms = (ctypes.c_double * count)()
        launches = (ctypes.c_uint64 * count)()
        lib.evo_b200_context_profile_read(self.handle, ms, launches, count)
        return {lib.evo_b200_profile_category_name(i).decode(): (ms[i], int(launches[i]))
                for i in range(count)}

    def slice_embed(self, device_tokens: int, row_begin: int, rows: int) -> None:
        self.library.check(self.library.lib.evo_b200_context_slice_embed(self.handle, device_tokens, row_begin, rows))

    def slice_run(self, row_begin: int, rows: int) -> None:
        self.library.check(self.library.lib.evo_b200_context_slice_run(self.handle, row_begin, rows))

    def slice_head(self, row_begin: int, rows: int) -> int:
        out = ctypes.c_void_p()
        self.library.check(self.library.lib.evo_b200_context_slice_head(self.handle, row_begin, rows,
                                                                        ctypes.byref(out)))
        return out.value

    def slice_hidden(self) -> int:
        return self.library.lib.evo_b200_context_slice_hidden(self.handle)

    def stages(self) -> list[StageInfo]:
        lib = self.library.lib
        result = []
        for index in range(lib.evo_b200_context_stage_count(self.handle)):
            info = StageInfo()
            info.struct_size = ctypes.sizeof(StageInfo)
            self.library.check(lib.evo_b200_context_stage_info(self.handle, index, ctypes.byref(info)))
            result.append(info)
        return result


class Sampler:
    def __init__(self, library: EvoLibrary, *, temperature=1.0, top_k=1, top_p=1.0, seed=0):
        self.library = library
        params = library.lib.evo_sampler_default_params()
        params.temperature, params.top_k, params.top_p, params.seed = temperature, top_k, top_p, seed
        self.handle = ctypes.c_void_p()
        library.check(library.lib.evo_sampler_create(ctypes.byref(params), ctypes.byref(self.handle)))

    def sample(self, logits: np.ndarray) -> int:
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        token = ctypes.c_uint32()
        self.library.check(self.library.lib.evo_sampler_sample(
            self.handle, logits.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), logits.size,
            ctypes.byref(token)))
        return token.value

    def close(self) -> None:
        if self.handle:
            self.library.lib.evo_sampler_free(self.handle)
            self.handle = None
