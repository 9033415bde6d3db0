"""Seeded synthetic decoder modules with the shapes the benchmark configurations name.

The reference's whole-model gates load ``models/gemma-3-*-ONNX`` files
(README.md:169-182) that are not available offline; these builders emit the same
kind of module the reference's lowering produces for such an export — the
composites ``SimplifiedLayerNormalization``, ``com.microsoft.MatMulNBits``,
``com.microsoft.GroupQueryAttention`` (with ``do_rotary``), ``Gelu`` — with
random-init weights. Module I/O follows what ``LlmSession`` feeds
(crates/onyxia-cli/src/llm.rs:115-182): ``input_ids``, ``attention_mask`` (all
ones, ``seqlens_k`` is derived from it like the exports do),
``past_key_values.N.{key,value}`` → ``logits``, ``present.N.{key,value}``.
"""
from __future__ import annotations

import dataclasses
import zlib

import numpy as np

from . import ir
from .ir import HostTensor


@dataclasses.dataclass
class DecoderConfig:
    name: str
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    act_dtype: int = ir.F16          # activations, scales, KV cache, embedding table
    eps: float = 1e-6
    rope_theta: float = 10000.0
    max_positions: int = 4096
    window: int = -1                 # local_window_size of local layers (−1: every layer is global)
    global_every: int = 0            # layer ℓ is global iff (ℓ+1) % global_every == 0 (0: all global)
    explicit_zero_points: bool = False   # pass a U4 zero-point tensor (all 8) instead of the default
    sandwich_norms: bool = False     # Gemma-3 post-attention / post-FFN norms before the residual adds
    last_logits_only: bool = False   # slice the last position before lm_head
    gelu_tanh: bool = True
    scale_range: tuple = (0.005, 0.02)   # uniform range of the int4 block scales

    @property
    def np_act(self):
        return np.float16 if self.act_dtype == ir.F16 else np.float32

    def layer_window(self, layer: int) -> int:
        if self.window < 0:
            return -1
        if self.global_every and (layer + 1) % self.global_every == 0:
            return -1
        return self.window

    def weight_bytes_per_token(self) -> int:
        """Packed int4 weights + scales read by one batch-1 decode step (algorithmic bytes)."""
        sb = 2 if self.act_dtype == ir.F16 else 4
        zp = 0.5 if self.explicit_zero_points else 0

        def mat(k, n):
            nb = (k + 31) // 32
            return int(n * nb * (16 + sb + zp))

        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        per_layer = (mat(self.hidden, q) + 2 * mat(self.hidden, kv) + mat(q, self.hidden) +
                     2 * mat(self.hidden, self.ffn) + mat(self.ffn, self.hidden))
        return self.layers * per_layer + mat(self.hidden, self.vocab)

    def kv_bytes_per_token(self, context: int) -> int:
        """K and V rows a batch-1 decode step reads at the given context length."""
        esz = 2 if self.act_dtype == ir.F16 else 4
        total = 0
        for l in range(self.layers):
            w = self.layer_window(l)
            rows = context + 1 if w < 0 else min(context + 1, w + 1)
            total += 2 * self.kv_heads * rows * self.head_dim * esz
        return total


# The benchmark configurations.
def config_c1() -> DecoderConfig:
    """2-layer Gemma-style decoder, fp32 activations/scales, explicit zero points."""
    return DecoderConfig("c1-2layer", layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64, ffn=2048, vocab=32000,
                         act_dtype=ir.F32, eps=1e-6, max_positions=256, explicit_zero_points=True)


def config_gemma3_1b() -> DecoderConfig:
    """Gemma-3-1B architecture: 26 layers, 5 local (window 512) : 1 global."""
    return DecoderConfig("gemma3-1b-arch-int4", layers=26, hidden=1152, heads=4, kv_heads=1, head_dim=256, ffn=6912,
                         vocab=262144, act_dtype=ir.F16, max_positions=2048, window=512, global_every=6,
                         sandwich_norms=True, last_logits_only=True)


def config_gemma3_27b() -> DecoderConfig:
    """Gemma-3-27B architecture: 62 layers, 5 local (window 1024) : 1 global."""
    return DecoderConfig("gemma3-27b-arch-int4", layers=62, hidden=5376, heads=32, kv_heads=16, head_dim=128, ffn=21504,
                         vocab=262144, act_dtype=ir.F16, max_positions=4096, window=1024, global_every=6,
                         sandwich_norms=True, last_logits_only=True)


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.default_rng([seed, zlib.crc32(name.encode())])


def rope_caches(cfg: DecoderConfig):
    half = cfg.head_dim // 2
    inv = cfg.rope_theta ** (-np.arange(half, dtype=np.float64) * 2.0 / cfg.head_dim)
    ang = np.arange(cfg.max_positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(cfg.np_act), np.sin(ang).astype(cfg.np_act)


def nbits_arrays(cfg: DecoderConfig, seed: int, name: str, k: int, n: int):
    """The seeded int4 weight `name`: (packed nibbles u8 [n·nb·16], scales [n·nb], packed zero points u8 or None)."""
    nb = (k + 31) // 32
    r = _rng(seed, name)
    packed = r.integers(0, 256, size=n * nb * 16, dtype=np.uint8)  # nibbles uniform over 0..15
    scales = r.uniform(cfg.scale_range[0], cfg.scale_range[1], size=n * nb).astype(cfg.np_act)
    zp = np.full((n * nb + 1) // 2, 0x88, dtype=np.uint8) if cfg.explicit_zero_points else None
    return packed, scales, zp


def norm_array(cfg: DecoderConfig, seed: int, name: str, width: int):
    return (1.0 + 0.02 * _rng(seed, name).standard_normal(width)).astype(cfg.np_act)


def embed_array(cfg: DecoderConfig, seed: int):
    return (0.02 * _rng(seed, "embed").standard_normal((cfg.vocab, cfg.hidden), dtype=np.float32)).astype(cfg.np_act)


class _Weights:
    """Adds seeded constants to a builder; big tensors are borrowed, not copied."""

    def __init__(self, b: ir.GraphBuilder, cfg: DecoderConfig, seed: int):
        self.b, self.cfg, self.seed = b, cfg, seed

    def nbits(self, name: str, k: int, n: int):
        nb = (k + 31) // 32
        packed, scales, zp = nbits_arrays(self.cfg, self.seed, name, k, n)
        w = self.b.constant(HostTensor(ir.U4, [n, nb, 32], packed), borrow=True)
        s = self.b.constant(HostTensor.from_numpy(scales), borrow=True)
        ins = [w, s]
        if zp is not None:
            ins.append(self.b.constant(HostTensor(ir.U4, [n, nb], zp), borrow=True))
        return ins

    def norm(self, name: str, width: int):
        return self.b.constant(HostTensor.from_numpy(norm_array(self.cfg, self.seed, name, width)))


def build_decoder(cfg: DecoderConfig, seed: int = 0) -> ir.Module:
    b = ir.GraphBuilder()
    W = _Weights(b, cfg, seed)
    adt = cfg.act_dtype
    B, S = b.sym("batch_size"), b.sym("sequence_length")
    P, T = b.sym("past_sequence_length"), b.sym("total_sequence_length")
    H, D, NH, KV = cfg.hidden, cfg.head_dim, cfg.heads, cfg.kv_heads

    ids = b.input("input_ids", ir.I64, [B, S])
    mask = b.input("attention_mask", ir.I64, [B, T])
    pasts = []
    for l in range(cfg.layers):
        pasts.append((b.input(f"past_key_values.{l}.key", adt, [B, KV, P, D]),
                      b.input(f"past_key_values.{l}.value", adt, [B, KV, P, D])))
    b.constrain(T, P + S, "GroupQueryAttention 'total_sequence_length' must equal the past KV length plus the new "
                          "sequence length")

    def nbits(x, name, k, n):
        b.set_loc(name, "MatMulNBits")
        return b.composite("com.microsoft.MatMulNBits", {"K": k, "N": n, "bits": 4, "block_size": 32},
                           [x] + W.nbits(name, k, n), [(adt, [B, S, n])])[0]

    def norm(x, name, shape=None):
        b.set_loc(name, "SimplifiedLayerNormalization")
        return b.composite("SimplifiedLayerNormalization", {"epsilon": float(cfg.eps), "axis": -1},
                           [x, W.norm(name, H)], [(adt, shape or [B, S, H])])[0]

    # seqlens_k = sum(attention_mask) − 1 as int32, the way the exports derive it
    b.set_loc("/model/attn_mask_reformat/seqlens", "ReduceSum")
    lens = b.reduce(ir.SUM, mask, [1], False)
    seqlens = b.cast(b.sub(lens, b.const_i64([1], [1])), ir.I32)

    cos_np, sin_np = rope_caches(cfg)
    cos = b.constant(HostTensor.from_numpy(cos_np))
    sin = b.constant(HostTensor.from_numpy(sin_np))

    b.set_loc("/model/embed_tokens/Gather", "Gather")
    x = b.gather(b.constant(HostTensor.from_numpy(embed_array(cfg, seed)), borrow=True), ids, 0)

    presents = []
    for l in range(cfg.layers):
        pre = f"/model/layers.{l}"
        h = norm(x, f"{pre}/input_layernorm")
        q = nbits(h, f"{pre}/attn/q_proj", H, NH * D)
        k = nbits(h, f"{pre}/attn/k_proj", H, KV * D)
        v = nbits(h, f"{pre}/attn/v_proj", H, KV * D)
        b.set_loc(f"{pre}/attn/GroupQueryAttention", "GroupQueryAttention")
        attn, pk, pv = b.composite(
            "com.microsoft.GroupQueryAttention",
            {"num_heads": NH, "kv_num_heads": KV, "scale": 0.0, "local_window_size": cfg.layer_window(l),
             "do_rotary": 1, "rotary_interleaved": 0, "has_attention_bias": 0},
            [q, k, v, pasts[l][0], pasts[l][1], seqlens, cos, sin],
            [(adt, [B, S, NH * D]), (adt, [B, KV, P + S, D]), (adt, [B, KV, P + S, D])])
        presents.append((pk, pv))
        o = nbits(attn, f"{pre}/attn/o_proj", NH * D, H)
        if cfg.sandwich_norms:
            o = norm(o, f"{pre}/post_attention_layernorm")
        b.set_loc(f"{pre}/residual_add_1", "Add")
        x = b.add(x, o)
        h2 = norm(x, f"{pre}/pre_feedforward_layernorm")
        gate = nbits(h2, f"{pre}/mlp/gate_proj", H, cfg.ffn)
        up = nbits(h2, f"{pre}/mlp/up_proj", H, cfg.ffn)
        b.set_loc(f"{pre}/mlp/act_fn/Gelu", "Gelu")
        act = b.composite("Gelu", {"approximate": "tanh" if cfg.gelu_tanh else "none"}, [gate], [(adt, [B, S, cfg.ffn])])[0]
        b.set_loc(f"{pre}/mlp/Mul", "Mul")
        m = b.mul(act, up)
        down = nbits(m, f"{pre}/mlp/down_proj", cfg.ffn, H)
        if cfg.sandwich_norms:
            down = norm(down, f"{pre}/post_feedforward_layernorm")
        b.set_loc(f"{pre}/residual_add_2", "Add")
        x = b.add(x, down)

    x = norm(x, "/model/norm")
    if cfg.last_logits_only:
        b.set_loc("/model/last_token/Slice", "Slice")
        x = b.slice(x, [(1, S - 1, S, 1)])
        b.set_loc("/lm_head/MatMulNBits", "MatMulNBits")
        logits = b.composite("com.microsoft.MatMulNBits", {"K": H, "N": cfg.vocab, "bits": 4, "block_size": 32},
                             [x] + W.nbits("/lm_head", H, cfg.vocab), [(adt, [B, 1, cfg.vocab])])[0]
    else:
        logits = nbits(x, "/lm_head", H, cfg.vocab)
    b.set_loc(None)
    b.output("logits", logits)
    for l, (pk, pv) in enumerate(presents):
        b.output(f"present.{l}.key", pk)
        b.output(f"present.{l}.value", pv)
    return b.finish()


def build_matmul_nbits(m: int, k: int, n: int, act_dtype: int = ir.F16, seed: int = 0, with_zp: bool = False):
    """Single-node module of the MatMulNBits sweep; returns (module, activation HostTensor)."""
    cfg = DecoderConfig("nbits", 0, 0, 0, 0, 0, 0, 0, act_dtype=act_dtype, explicit_zero_points=with_zp)
    b = ir.GraphBuilder()
    W = _Weights(b, cfg, seed)
    a = b.input("a", act_dtype, [m, k])
    ins = W.nbits(f"w{k}x{n}", k, n)
    if with_zp:  # random zero points exercise the 4-input form
        nb = (k + 31) // 32
        zp = _rng(seed, "zp").integers(0, 256, size=(n * nb + 1) // 2, dtype=np.uint8)
        ins[2] = b.constant(HostTensor(ir.U4, [n, nb], zp))
    y = b.composite("com.microsoft.MatMulNBits", {"K": k, "N": n, "bits": 4, "block_size": 32}, [a] + ins,
                    [(act_dtype, [m, n])])[0]
    b.output("y", y)
    act = _rng(seed, "act").standard_normal((m, k)).astype(cfg.np_act)
    return b.finish(), HostTensor.from_numpy(act)


def build_gqa(batch: int, heads: int, kv_heads: int, head_dim: int, past: int, seq: int = 1, act_dtype: int = ir.F16,
              window: int = -1, rotary: bool = True, seed: int = 0, max_positions: int | None = None):
    """Single GroupQueryAttention node with dense seqlens (= past + seq − 1); returns (module, feed dict)."""
    np_act = np.float16 if act_dtype == ir.F16 else np.float32
    b = ir.GraphBuilder()
    q = b.input("q", act_dtype, [batch, seq, heads * head_dim])
    k = b.input("k", act_dtype, [batch, seq, kv_heads * head_dim])
    v = b.input("v", act_dtype, [batch, seq, kv_heads * head_dim])
    pk = b.input("past_key", act_dtype, [batch, kv_heads, past, head_dim])
    pv = b.input("past_value", act_dtype, [batch, kv_heads, past, head_dim])
    sl = b.input("seqlens_k", ir.I32, [batch])
    ins = [q, k, v, pk, pv, sl]
    if rotary:
        cfg = DecoderConfig("gqa", 0, 0, heads, kv_heads, head_dim, 0, 0, act_dtype=act_dtype,
                            max_positions=max_positions or (past + seq))
        c, s = rope_caches(cfg)
        ins += [b.constant(HostTensor.from_numpy(c)), b.constant(HostTensor.from_numpy(s))]
    total = past + seq
    outs = b.composite("com.microsoft.GroupQueryAttention",
                       {"num_heads": heads, "kv_num_heads": kv_heads, "scale": 0.0, "local_window_size": window,
                        "do_rotary": int(rotary), "rotary_interleaved": 0, "has_attention_bias": 0}, ins,
                       [(act_dtype, [batch, seq, heads * head_dim]), (act_dtype, [batch, kv_heads, total, head_dim]),
                        (act_dtype, [batch, kv_heads, total, head_dim])])
    b.output("out", outs[0])
    b.output("present_key", outs[1])
    b.output("present_value", outs[2])
    r = _rng(seed, "gqa")
    feed = {
        "q": HostTensor.from_numpy(r.standard_normal((batch, seq, heads * head_dim)).astype(np_act)),
        "k": HostTensor.from_numpy(r.standard_normal((batch, seq, kv_heads * head_dim)).astype(np_act)),
        "v": HostTensor.from_numpy(r.standard_normal((batch, seq, kv_heads * head_dim)).astype(np_act)),
        "past_key": HostTensor.from_numpy(r.standard_normal((batch, kv_heads, past, head_dim)).astype(np_act)),
        "past_value": HostTensor.from_numpy(r.standard_normal((batch, kv_heads, past, head_dim)).astype(np_act)),
        "seqlens_k": HostTensor.from_numpy(np.full(batch, total - 1, dtype=np.int32)),
    }
    return b.finish(), feed
