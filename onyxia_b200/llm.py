"""KV-cache generation loop over a prepared session ≙ ``LlmSession``
(crates/onyxia-cli/src/llm.rs:26-246).

Generic over the backend session: anything with ``upload`` / ``run`` /
``download`` (the CUDA session, or the CPU oracle's session in tests).
``present.*`` output handles are stored and fed back as ``past_key_values.*``
inputs of the next call; only the logits (or, with ``greedy_on_device``, the
8-byte argmax) cross back to the host.
"""
from __future__ import annotations

import numpy as np

from . import ir
from .ir import HostTensor, Module


def discover_kv_pairs(module: Module) -> list:
    """``present.N.*`` outputs paired with ``past_key_values.N.*`` inputs (llm.rs:232-246)."""
    inputs = set(module.input_names())
    pairs = []
    for out in module.output_names():
        if out.startswith("present."):
            past = "past_key_values." + out[len("present."):]
            if past in inputs:
                pairs.append((out, past))
    return pairs


class LlmSession:
    def __init__(self, backend, module: Module, max_seq_len: int):
        # everything needed later is read before prepare() consumes the module (llm.rs:43-61)
        self.input_names = module.input_names()
        self.input_desc = [module.input_desc(i) for i in range(len(self.input_names))]
        self._shape_module = module.clone()  # graph only; constant bytes are shared, not copied
        self.kv_pairs = discover_kv_pairs(module)
        self.session = backend.prepare(module)
        self.kv_cache: dict = {}
        self.past_seq_len = 0
        self.max_seq_len = max_seq_len
        self._np = {ir.F32: np.float32, ir.F16: np.float16, ir.I64: np.int64, ir.I32: np.int32}

    def _bindings(self, seq: int) -> dict:
        return {"batch_size": 1, "sequence_length": seq, "past_sequence_length": self.past_seq_len,
                "total_sequence_length": self.past_seq_len + seq}

    def prefill(self, input_ids) -> np.ndarray:
        ids = list(input_ids)
        if not ids:
            raise ValueError("Cannot prefill with empty input_ids")
        if len(ids) > self.max_seq_len:
            raise ValueError(f"Input length {len(ids)} exceeds max_seq_len {self.max_seq_len}")
        return self.step(ids, list(range(len(ids))))

    def decode(self, token_id: int) -> np.ndarray:
        if self.past_seq_len >= self.max_seq_len:
            raise ValueError(f"Sequence length {self.past_seq_len + 1} would exceed max_seq_len {self.max_seq_len}")
        return self.step([int(token_id)], [self.past_seq_len])

    def _inputs(self, ids, positions):
        seq = len(ids)
        bindings = self._bindings(seq)
        feed = []
        for i, name in enumerate(self.input_names):
            dtype, _ = self.input_desc[i]
            if name == "input_ids":
                t = ids if not isinstance(ids, list) else self.session.upload(
                    HostTensor.from_numpy(np.asarray(ids, dtype=np.int64).reshape(1, seq)))
            elif name == "position_ids":
                t = self.session.upload(HostTensor.from_numpy(np.asarray(positions, dtype=np.int64).reshape(1, seq)))
            elif name.startswith("past_key_values.") and name in self.kv_cache:
                t = self.kv_cache[name]
            else:
                dims = self._shape_module.eval_input_shape(i, bindings)
                if dtype not in self._np:
                    raise ValueError(f"input '{name}' has unsupported dtype {ir.DTYPE_NAMES[dtype]}")
                # empty cache on the first step; masks and friends are all ones (llm.rs:136-151)
                fill = np.zeros if name.startswith("past_key_values.") else np.ones
                t = self.session.upload(HostTensor.from_numpy(fill(dims, dtype=self._np[dtype])))
            feed.append((name, t))
        return feed, seq

    def _advance(self, outputs, seq):
        by_name = dict(outputs)
        for present, past in self.kv_pairs:
            if present not in by_name:
                raise KeyError(f"output '{present}' missing")
            self.kv_cache[past] = by_name[present]
        self.past_seq_len += seq
        if "logits" not in by_name:
            raise KeyError("output 'logits' missing")
        return by_name["logits"]

    def step(self, ids, positions) -> np.ndarray:
        """One forward pass; returns the logits of the last position as f32 [vocab] (llm.rs:110-183)."""
        feed, seq = self._inputs(ids, positions)
        logits = self._advance(self.session.run(feed), seq)
        host = self.session.download(logits).numpy()
        return host.reshape(-1, host.shape[-1])[-1].astype(np.float32)

    def step_greedy(self, ids, positions) -> int:
        """Same pass, but the argmax runs on the device and 8 bytes come back."""
        feed, seq = self._inputs(ids, positions)
        logits = self._advance(self.session.run(feed), seq)
        tok = self.session.download(self.session.argmax_last(logits)).numpy()
        return int(tok.reshape(-1)[-1])

    def reset(self) -> None:
        self.past_seq_len = 0

    def reset_full(self) -> None:
        self.past_seq_len = 0
        self.kv_cache.clear()

    def sequence_length(self) -> int:
        return self.past_seq_len


def sample_greedy(logits: np.ndarray) -> int:
    """Highest logit; among equal maxima the last one, like ``Iterator::max_by``
    (crates/onyxia-cli/src/sampling.rs:71-80)."""
    logits = np.asarray(logits)
    if logits.size == 0:
        raise ValueError("Cannot sample_greedy from empty logits")
    return int(logits.size - 1 - np.argmax(logits[::-1]))


class NativeLlmSession:
    """The same loop run natively by the CUDA library (`ox_llm_*`): one call per step, greedy choice
    on the device. Use it where the per-step host overhead matters; `LlmSession` stays the generic form
    that also drives the CPU oracle."""

    def __init__(self, backend, module: Module, max_seq_len: int):
        import ctypes as C
        from . import _ffi
        self._C, self._lib = C, _ffi.cuda_lib()
        self.session = backend.prepare(module)
        h = C.c_void_p()
        _ffi.check(self._lib.ox_llm_create(self.session._h, max_seq_len, C.byref(h)))
        self._h = h

    def step_greedy(self, ids) -> int:
        C = self._C
        from . import _ffi
        arr = (C.c_int64 * len(ids))(*ids)
        tok = C.c_int64()
        _ffi.check(self._lib.ox_llm_step(self._h, arr, len(ids), C.byref(tok), None, 0, None))
        return tok.value

    def generate(self, ids, n_new: int) -> list:
        """`n_new` greedy tokens after `ids`; the token id travels from step to step on the device (ox_llm_generate)."""
        C = self._C
        from . import _ffi
        arr = (C.c_int64 * len(ids))(*ids)
        out = (C.c_int64 * max(n_new, 1))()
        _ffi.check(self._lib.ox_llm_generate(self._h, arr, len(ids), int(n_new), out))
        return [int(out[i]) for i in range(n_new)]

    def step_sampled(self, ids, temperature: float, top_k: int, top_p: float, uniform: float) -> int:
        """The step with the next token drawn on the device (≙ sampling::sample, crates/onyxia-cli/src/sampling.rs:36-65);
        `uniform` is the caller's random number in [0, 1]."""
        C = self._C
        from . import _ffi
        arr = (C.c_int64 * len(ids))(*ids)
        tok = C.c_int64()
        _ffi.check(self._lib.ox_llm_step_sampled(self._h, arr, len(ids), float(temperature), int(top_k), float(top_p), float(uniform),
                                                 C.byref(tok)))
        return tok.value

    def step_logits(self, ids) -> np.ndarray:
        C = self._C
        from . import _ffi
        arr = (C.c_int64 * len(ids))(*ids)
        buf = np.empty(1 << 20, dtype=np.uint8)
        written = C.c_size_t()
        _ffi.check(self._lib.ox_llm_step(self._h, arr, len(ids), None, buf.ctypes.data_as(C.c_void_p), buf.size, C.byref(written)))
        raw = buf[:written.value]
        np_dt = np.float16 if self._lib.ox_llm_logits_dtype(self._h) == ir.F16 else np.float32
        return raw.view(np_dt).astype(np.float32)

    def sequence_length(self) -> int:
        return self._lib.ox_llm_sequence_length(self._h)

    def reset(self) -> None:
        self._lib.ox_llm_reset(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.ox_llm_free(self._h)
            self._h = None
