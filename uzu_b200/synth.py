"""Synthetic uzu-format checkpoints (config.json + model.safetensors) for tests and benchmarks.

There is no network in the build/bench environment, so real checkpoints cannot be fetched; this
module emits seeded random weights in exactly the on-disk layout the reference engine loads
(SURVEY.md Appendix A): config.json follows crates/backend-uzu/src/config/** (abstract-config
variants carry a "type" tag, every Option field is present as null), tensor keys follow
encodable_block/{embedding,transformer_layer,mixer/attention/mod,mixer/delta_net,mlp/mod}.rs and
per-matrix quantisation specs are JSON strings under `<prefix>.spec` in the safetensors
`__metadata__` (parameters/loader.rs:219-228).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path

import numpy as np

from . import safetensors_io as st


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bits (same as `half::bf16::from_f32`)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    up = ((u & np.uint32(0x8000)) != 0) & ((u & np.uint32(0x17FFF)) != 0)
    return ((u >> 16) + up.astype(np.uint32)).astype(np.uint16)


@dataclass
class QuantSpec:
    kind: str = "int"          # "int" (IntSpec), "mlx" (MLXSpec), "fp" (FullPrecisionSpec)
    bits: int = 4
    group_size: int = 64
    symmetric: bool = False    # IntSpec.is_symmetric
    rht: bool = False          # HybridSpec: 32-wide input/output randomized Hadamard around this quantization (Mirai RHT)

    def spec_json(self, layout: str) -> dict:
        if self.rht:
            inner = QuantSpec(self.kind, self.bits, self.group_size, self.symmetric).spec_json(layout)
            return {"type": "HybridSpec", "quantization_spec": inner, "adapter_spec": None, "incoherence_block_size": 32,
                    "incoherence_processing_mode": "input_output"}
        if self.kind == "fp":
            return {"type": "FullPrecisionSpec", "layout": layout}
        if self.kind == "mlx":
            return {"type": "MLXSpec", "bits": self.bits, "group_size": self.group_size, "layout": layout}
        return {"type": "IntSpec", "bits": self.bits, "group_size": self.group_size,
                "is_symmetric": self.symmetric, "layout": layout}


@dataclass
class ModelSpec:
    name: str
    model_dim: int
    hidden_dim: int
    vocab_size: int
    # per layer: "attn" or "delta"
    layer_kinds: list = field(default_factory=list)
    num_heads: int = 8
    num_groups: int = 2
    head_dim: int = 128
    rope: dict = field(default_factory=dict)      # AnyRoPEConfig json (with "type")
    qk_norm: bool = False
    qk_norm_scale_offset: float | None = None
    attn_gate: bool = False
    norm_eps: float = 1e-5
    norm_scale_offset: float | None = None
    upcast_mode: str = "only_normalization"
    tied_embeddings: bool = False
    quant: QuantSpec = field(default_factory=QuantSpec)
    embedding_quant: QuantSpec | None = None      # default: same as `quant`
    # DeltaNet
    dn_num_heads: int = 16
    dn_num_groups: int = 16
    dn_head_dim: int = 128
    dn_value_head_dim: int = 128
    dn_kernel_size: int = 4
    max_sequence_length: int = 8192

    @property
    def num_layers(self) -> int:
        return len(self.layer_kinds)


def _norm_cfg(spec: ModelSpec, scale_offset=None, eps=None):
    return {"epsilon": eps if eps is not None else spec.norm_eps,
            "scale_offset": scale_offset if scale_offset is not None else spec.norm_scale_offset,
            "upcast_mode": spec.upcast_mode, "subtract_mean": False, "has_scale": True, "has_biases": False}


def build_config(spec: ModelSpec) -> dict:
    layers = []
    for kind in spec.layer_kinds:
        if kind == "attn":
            mixer = {
                "type": "AttentionConfig", "qkv_projection_config": {}, "out_projection_config": {},
                "query_norm_config": _norm_cfg(spec, spec.qk_norm_scale_offset, 1e-6) if spec.qk_norm else None,
                "key_norm_config": _norm_cfg(spec, spec.qk_norm_scale_offset, 1e-6) if spec.qk_norm else None,
                "num_heads": spec.num_heads, "num_groups": spec.num_groups, "head_dim": spec.head_dim,
                "is_causal": True, "scale": None, "sliding_window_size": None, "logit_soft_cap": None,
                "has_sinks": False, "has_qkv_biases": False, "has_out_biases": False,
                "gate_projection_config": {} if spec.attn_gate else None, "normalize_values": False,
                "is_kv_sharing": False,
            }
            rope = dict(spec.rope)
        else:
            mixer = {
                "type": "DeltaNetConfig", "in_proj_config": {}, "conv_config": {"has_biases": False},
                "out_proj_config": {}, "norm_config": _norm_cfg(spec, None, 1e-6),
                "num_heads": spec.dn_num_heads, "num_groups": spec.dn_num_groups, "head_dim": spec.dn_head_dim,
                "value_head_dim": spec.dn_value_head_dim, "kernel_size": spec.dn_kernel_size,
            }
            rope = None
        layers.append({
            "pre_mixer_norm_config": _norm_cfg(spec), "mixer_config": mixer, "post_mixer_norm_config": None,
            "pre_mlp_norm_config": _norm_cfg(spec),
            "mlp_config": {"type": "DenseMLPConfig", "linear_config": {}, "activation": {"type": "SiLU", "alpha": 1.0},
                           "has_up_biases": False, "has_down_biases": False, "gate_clipping": None,
                           "up_clipping": None},
            "post_mlp_norm_config": None, "hidden_dim": None, "ple_config": None, "has_post_layer_scalar": False,
            "kv_source_layer_index": None, "rope_config": rope,
        })
    emb_type = "TiedEmbeddingConfig" if spec.tied_embeddings else "UntiedEmbeddingConfig"
    return {
        "type": "LanguageModelConfig",
        "token_codec_config": {"type": "RawTextCodecConfig"},
        "decoder_config": {
            "embedding_config": {"type": emb_type, "input_scale": None, "logit_soft_cap": None, "logit_scale": None},
            "transformer_config": {"layer_configs": layers, "output_norm_config": _norm_cfg(spec),
                                   "model_dim": spec.model_dim, "hidden_dim": spec.hidden_dim},
            "vocab_size": spec.vocab_size, "ple_model_config": None, "embedding_norm_config": None,
        },
        "generation_config": {"stop_token_ids": [], "temperature": None, "top_k": None, "top_p": None, "min_p": None,
                              "banned_tokens": None, "repetition_penalty": None, "presence_penalty": None,
                              "frequency_penalty": None, "suffix_repetition_length": None},
    }


# ---------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------
def quantized_matrix(rng: np.random.Generator, rows: int, cols: int, q: QuantSpec, target_std: float):
    """Random block-quantised [rows, cols] matrix in uzu layout.

    codes uniform in [0, 2^bits); packed little-endian nibbles / bytes row-major
    (cpu/kernel/matmul/kernel.rs:236-243); scales bf16 [rows, cols/gs]; zero points nibble-packed
    [rows, ceil(groups/2)] (4-bit) or [rows, groups] (8-bit) (weight_matrix.rs:136-151).
    """
    out = {}
    if q.kind == "fp":
        w = rng.standard_normal((rows, cols), dtype=np.float32) * target_std
        out["weights"] = st.as_bf16(f32_to_bf16_bits(w))
        return out
    levels = 1 << q.bits
    groups = -(-cols // q.group_size)
    if q.bits == 4:
        packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    else:
        packed = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
    out["weights"] = packed
    # (code - zp) has std ~ levels/sqrt(6); choose scales so dequantised weights have ~target_std
    base = target_std / (levels / np.sqrt(6.0))
    scales = (rng.random((rows, groups), dtype=np.float32) + 0.5) * base
    out["scales"] = st.as_bf16(f32_to_bf16_bits(scales))
    if q.kind == "mlx":
        sc = st_bits_to_f32(out["scales"])
        zp = rng.integers(0, levels, size=(rows, groups)).astype(np.float32)
        out["biases"] = st.as_bf16(f32_to_bf16_bits(-sc * zp))
    elif not q.symmetric:
        if q.bits == 4:
            out["zero_points"] = rng.integers(0, 256, size=(rows, -(-groups // 2)), dtype=np.uint8)
        else:
            out["zero_points"] = rng.integers(0, 256, size=(rows, groups), dtype=np.uint8)
    return out


def st_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _add_matrix(tensors, meta, prefix, rng, rows, cols, q, layout, target_std):
    if q.rht:
        # RHTLinearWrapper::load_inner_with_output_rht (linear/rht_wrapper.rs:141-176): i32 +-1 signs + the inner matrix under `quantized`
        assert layout == "output_input" and q.kind != "fp" and rows % 32 == 0 and cols % 32 == 0
        inner = QuantSpec(q.kind, q.bits, q.group_size, q.symmetric)
        tensors[f"{prefix}.incoherence_signs.input_signs"] = rng.choice(np.array([-1, 1], np.int32), cols)
        tensors[f"{prefix}.incoherence_signs.output_signs"] = rng.choice(np.array([-1, 1], np.int32), rows)
        _add_matrix(tensors, meta, prefix + ".quantized", rng, rows, cols, inner, layout, target_std)
        meta[f"{prefix}.spec"] = json.dumps(q.spec_json(layout))
        return
    for k, v in quantized_matrix(rng, rows, cols, q, target_std).items():
        tensors[f"{prefix}.{k}"] = v
    meta[f"{prefix}.spec"] = json.dumps(q.spec_json(layout))


def build_weights(spec: ModelSpec, seed: int = 0):
    rng = np.random.default_rng(seed)
    T, M = {}, {}
    H, F, V = spec.model_dim, spec.hidden_dim, spec.vocab_size
    eq = spec.embedding_quant or spec.quant
    if eq.rht:     # quantized embeddings with a Hadamard are unimplemented on the reference CPU backend (quant_embedding.rs:32-34)
        eq = QuantSpec(eq.kind, eq.bits, eq.group_size, eq.symmetric)
    if spec.tied_embeddings:
        _add_matrix(T, M, "decoder.embedding.embedding", rng, V, H, eq, "input_output", 1.0 / np.sqrt(H) * 4.0)
    else:
        _add_matrix(T, M, "decoder.embedding.input_embedding", rng, V, H, eq, "input_output", 1.0)
        _add_matrix(T, M, "decoder.embedding.output_embedding", rng, V, H, eq, "input_output", 1.0 / np.sqrt(H) * 4.0)

    def norm_scales(n):
        base = 0.0 if spec.norm_scale_offset else 1.0
        return (base + rng.standard_normal(n, dtype=np.float32) * 0.02).astype(np.float32)

    for i, kind in enumerate(spec.layer_kinds):
        p = f"decoder.transformer.layers.{i}"
        T[f"{p}.pre_mixer_norm.scales"] = norm_scales(H)
        T[f"{p}.pre_mlp_norm.scales"] = norm_scales(H)
        if kind == "attn":
            qd = spec.num_heads * spec.head_dim
            kvd = spec.num_groups * spec.head_dim
            _add_matrix(T, M, f"{p}.mixer.qkv_projection.weights", rng, qd + 2 * kvd, H, spec.quant, "output_input",
                        1.0 / np.sqrt(H))
            if spec.qk_norm:
                off = 0.0 if spec.qk_norm_scale_offset else 1.0
                T[f"{p}.mixer.query_norm.scales"] = (off + rng.standard_normal(spec.head_dim, dtype=np.float32) * 0.05).astype(np.float32)
                T[f"{p}.mixer.key_norm.scales"] = (off + rng.standard_normal(spec.head_dim, dtype=np.float32) * 0.05).astype(np.float32)
            if spec.attn_gate:
                _add_matrix(T, M, f"{p}.mixer.gate_projection.weights", rng, qd, H, spec.quant, "output_input",
                            1.0 / np.sqrt(H))
            _add_matrix(T, M, f"{p}.mixer.out_projection.weights", rng, H, qd, spec.quant, "output_input",
                        1.0 / np.sqrt(qd))
        else:
            key_dim = spec.dn_num_groups * spec.dn_head_dim
            value_dim = spec.dn_num_heads * spec.dn_value_head_dim
            conv_dim = 2 * key_dim + value_dim
            total = conv_dim + value_dim + 2 * spec.dn_num_heads
            _add_matrix(T, M, f"{p}.mixer.in_proj.weights", rng, total, H, spec.quant, "output_input", 1.0 / np.sqrt(H))
            T[f"{p}.mixer.conv.weights"] = (rng.standard_normal((conv_dim, spec.dn_kernel_size), dtype=np.float32) * 0.5).astype(np.float32)
            T[f"{p}.mixer.a_log"] = rng.uniform(-1.0, 1.0, spec.dn_num_heads).astype(np.float32)
            T[f"{p}.mixer.dt_bias"] = rng.uniform(-1.0, 1.0, spec.dn_num_heads).astype(np.float32)
            T[f"{p}.mixer.norm.scales"] = (1.0 + rng.standard_normal(spec.dn_value_head_dim, dtype=np.float32) * 0.05).astype(np.float32)
            _add_matrix(T, M, f"{p}.mixer.out_proj.weights", rng, H, value_dim, spec.quant, "output_input",
                        1.0 / np.sqrt(value_dim))
        _add_matrix(T, M, f"{p}.mlp.up_projection.weights", rng, 2 * F, H, spec.quant, "output_input", 1.0 / np.sqrt(H))
        _add_matrix(T, M, f"{p}.mlp.down_projection.weights", rng, H, F, spec.quant, "output_input", 1.0 / np.sqrt(F))
    T["decoder.transformer.output_norm.scales"] = norm_scales(H)
    return T, M


def write_model(spec: ModelSpec, path, seed: int = 0) -> Path:
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(build_config(spec), indent=1))
    tensors, meta = build_weights(spec, seed)
    st.save(path / "model.safetensors", tensors, meta)
    (path / "synth_spec.json").write_text(json.dumps(asdict(spec), indent=1))
    return path


# ---------------------------------------------------------------------------------------------
# presets (BASELINE.json configs)
# ---------------------------------------------------------------------------------------------
LLAMA3_ROPE = {"type": "LlamaRoPEConfig", "base": 500000.0, "max_sequence_length": 8192, "head_dim": 128,
               "scaling_factor": 8.0, "original_context_length": 8192, "low_frequency_factor": 1.0,
               "high_frequency_factor": 4.0}


def llama3_8b(bits=4, group_size=64, layers=32) -> ModelSpec:
    return ModelSpec(name=f"llama3-8b-int{bits}", model_dim=4096, hidden_dim=14336, vocab_size=128256,
                     layer_kinds=["attn"] * layers, num_heads=32, num_groups=8, head_dim=128, rope=dict(LLAMA3_ROPE),
                     norm_eps=1e-5, quant=QuantSpec("int", bits, group_size, False))


def llama3_70b(bits=4, group_size=64, layers=80) -> ModelSpec:
    return ModelSpec(name=f"llama3-70b-int{bits}", model_dim=8192, hidden_dim=28672, vocab_size=128256,
                     layer_kinds=["attn"] * layers, num_heads=64, num_groups=8, head_dim=128, rope=dict(LLAMA3_ROPE),
                     norm_eps=1e-5, quant=QuantSpec("int", bits, group_size, False))


def qwen35_0p8b(bits=4, group_size=64, layers=24, hybrid=True, vocab=248320) -> ModelSpec:
    """Qwen3.5-0.8B: linear shapes pinned by the reference's bench table (tests/matmul/shape.rs:82-88);
    layer mix (3 DeltaNet : 1 attention), vocab and rotary fraction from the public HF config
    (not pinned in the reference). hybrid=False gives the dense-attention stand-in."""
    kinds = [("attn" if (i % 4 == 3) else "delta") for i in range(layers)] if hybrid else ["attn"] * layers
    rope = {"type": "UnscaledRoPEConfig", "base": 10000000.0, "max_sequence_length": 262144, "head_dim": 64}
    return ModelSpec(name=f"qwen3.5-0.8b-int{bits}" + ("" if hybrid else "-dense"), model_dim=1024, hidden_dim=3584,
                     vocab_size=vocab, layer_kinds=kinds, num_heads=8, num_groups=2, head_dim=256, rope=rope,
                     qk_norm=True, qk_norm_scale_offset=1.0, attn_gate=True, norm_eps=1e-6, norm_scale_offset=1.0,
                     tied_embeddings=True, quant=QuantSpec("int", bits, group_size, False),
                     dn_num_heads=16, dn_num_groups=16, dn_head_dim=128, dn_value_head_dim=128, dn_kernel_size=4,
                     max_sequence_length=262144)


def tiny(kind="llama", quant: QuantSpec | None = None, layers=2) -> ModelSpec:
    """Small models for tests: same structure, small dims."""
    quant = quant or QuantSpec("int", 4, 64, False)
    if kind == "llama":
        rope = dict(LLAMA3_ROPE, head_dim=64)
        return ModelSpec(name="tiny-llama", model_dim=256, hidden_dim=512, vocab_size=1000,
                         layer_kinds=["attn"] * layers, num_heads=4, num_groups=2, head_dim=64, rope=rope, quant=quant)
    if kind == "qwen-dense":
        rope = {"type": "UnscaledRoPEConfig", "base": 1e6, "max_sequence_length": 4096, "head_dim": 32}
        return ModelSpec(name="tiny-qwen-dense", model_dim=256, hidden_dim=512, vocab_size=1200,
                         layer_kinds=["attn"] * layers, num_heads=4, num_groups=2, head_dim=64, rope=rope,
                         qk_norm=True, qk_norm_scale_offset=1.0, attn_gate=True, norm_eps=1e-6, norm_scale_offset=1.0,
                         tied_embeddings=True, quant=quant)
    if kind == "qwen-hybrid":
        rope = {"type": "UnscaledRoPEConfig", "base": 1e6, "max_sequence_length": 4096, "head_dim": 32}
        kinds = [("attn" if (i % 2 == 1) else "delta") for i in range(layers)]
        return ModelSpec(name="tiny-qwen-hybrid", model_dim=256, hidden_dim=512, vocab_size=1200, layer_kinds=kinds,
                         num_heads=4, num_groups=2, head_dim=64, rope=rope, qk_norm=True, qk_norm_scale_offset=1.0,
                         attn_gate=True, norm_eps=1e-6, norm_scale_offset=1.0, tied_embeddings=True, quant=quant,
                         dn_num_heads=4, dn_num_groups=2, dn_head_dim=128, dn_value_head_dim=128, dn_kernel_size=4)
    if kind == "llama-512":        # dims that the fused decode kernels cover (k multiple of 512)
        rope = dict(LLAMA3_ROPE, head_dim=64)
        return ModelSpec(name="tiny-llama-512", model_dim=512, hidden_dim=1024, vocab_size=2048, layer_kinds=["attn"] * layers,
                         num_heads=8, num_groups=2, head_dim=64, rope=rope, quant=quant)
    if kind == "qwen-hybrid-512":
        rope = {"type": "UnscaledRoPEConfig", "base": 1e6, "max_sequence_length": 4096, "head_dim": 32}
        kinds = [("attn" if (i % 2 == 1) else "delta") for i in range(layers)]
        return ModelSpec(name="tiny-qwen-hybrid-512", model_dim=512, hidden_dim=1024, vocab_size=2048, layer_kinds=kinds,
                         num_heads=8, num_groups=2, head_dim=64, rope=rope, qk_norm=True, qk_norm_scale_offset=1.0, attn_gate=True,
                         norm_eps=1e-6, norm_scale_offset=1.0, tied_embeddings=True, quant=quant, dn_num_heads=4, dn_num_groups=4,
                         dn_head_dim=128, dn_value_head_dim=128, dn_kernel_size=4)
    raise ValueError(kind)


PRESETS = {"llama3-8b": llama3_8b, "llama3-70b": llama3_70b, "qwen3.5-0.8b": qwen35_0p8b}


# ---------------------------------------------------------------------------------------------
# Punilix (parallel-block family): config.json {"architecture": "Punilix", "width", "vocab", "norm": {"eps", "groups"},
# "logit_softcap", "layers": [{"type", "mixer", "mlp"}]}; tensors embed, head, final.norm, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*
# ---------------------------------------------------------------------------------------------
def punilix_delta_layer(heads: int, dim: int, mlp: dict | None) -> dict:
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def punilix_latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, mlp: dict | None, scale: float | None = None,
                         base: float = 10000.0, scaling: dict | None = None) -> dict:
    rot = {"base": base, "dims": rot_dim, "scaling": scaling}
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
                      "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)},
            "mlp": mlp}


def punilix_dense_mlp(ff: int, limit: float = 7.0) -> dict:
    return {"kind": "dense", "ff": ff, "limit": limit}


def punilix_moe_mlp(ff: int, experts: int, top: int, limit: float = 7.0) -> dict:
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def punilix_config(width: int, vocab: int, layers: list, norm_groups: int = 1, eps: float = 1e-5, logit_softcap: float | None = 30.0) -> dict:
    return {"architecture": "Punilix", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": norm_groups},
            "logit_softcap": logit_softcap, "layers": layers}


def punilix_tensors(config: dict, seed: int = 0, decay_rank: int = 16) -> dict:
    """Seeded random tensors of a Punilix config: float arrays are f32 values that bf16 holds exactly, tables are int32."""
    rng = np.random.default_rng(seed)
    W, V = config["width"], config["vocab"]

    def bf(x):
        return st_bits_to_f32(f32_to_bf16_bits(np.asarray(x, np.float32)))

    def mat(rows, cols, gain=1.0):
        return bf(rng.standard_normal((rows, cols), dtype=np.float32) * (gain / np.sqrt(cols)))

    def vec(n, mean=1.0, spread=0.1):
        return bf(mean + spread * rng.standard_normal(n, dtype=np.float32))

    t = {"embed": mat(V, W, np.sqrt(W)), "head": mat(V, W, 2.0), "final.norm": vec(W)}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        t[p + "norm1"] = vec(W)
        m = L["mixer"]
        if L["type"] == "general_delta":
            hd = m["heads"] * m["dim"]
            for nm in ("r", "k", "v", "g", "a"):
                t[p + "mix." + nm] = mat(hd, W)
            t[p + "mix.a.b"] = vec(hd, 0.0, 0.5)
            t[p + "mix.w1"] = mat(decay_rank, W)
            t[p + "mix.w2"] = mat(hd, decay_rank, 2.0)
            t[p + "mix.w0"] = vec(hd, -1.0, 1.5)
            t[p + "mix.norm"] = vec(hd)
            t[p + "mix.o"] = mat(W, hd)
        elif L["type"] == "latent_attention":
            H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"] = mat(Q, W)
            t[p + "mix.dq.norm"] = vec(Q)
            t[p + "mix.uq"] = mat(H * (dn + dr), Q, 2.0)
            t[p + "mix.dkv"] = mat(R + dr, W)
            t[p + "mix.dkv.norm"] = vec(R)
            t[p + "mix.uk"] = mat(H * dn, R, 2.0)
            t[p + "mix.uv"] = mat(H * dv, R)
            t[p + "mix.g"] = mat(H * dv, W)
            t[p + "mix.o"] = mat(W, H * dv)
        else:
            raise ValueError(L["type"])
        ml = L.get("mlp")
        if ml is None:
            continue
        if ml["kind"] == "dense":
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(ml["ff"], W, 2.0), mat(ml["ff"], W, 2.0), mat(W, ml["ff"])
        else:
            f, E, top = ml["expert"]["ff"], ml["router"]["experts"], ml["router"]["top"]
            for x in range(E):
                q = f"{p}mlp.e{x}."
                t[q + "gate"], t[q + "up"], t[q + "down"] = mat(f, W, 2.0), mat(f, W, 2.0), mat(W, f)
            t[p + "mlp.table"] = np.stack([rng.permutation(E)[:top] for _ in range(V)]).astype(np.int32)
    return t


def write_punilix_model(config: dict, path, seed: int = 0, tensors: dict | None = None) -> Path:
    """config.json + model.safetensors (bf16 floats, int32 tables). `tensors` overrides the seeded random ones (values are rounded to bf16)."""
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config, indent=1))
    tensors = tensors if tensors is not None else punilix_tensors(config, seed)
    out = {}
    for name, v in tensors.items():
        v = np.asarray(v)
        out[name] = np.ascontiguousarray(v, np.int32) if np.issubdtype(v.dtype, np.integer) else st.as_bf16(f32_to_bf16_bits(v.astype(np.float32)).reshape(v.shape))
    st.save(path / "model.safetensors", out)
    return path


def punilix_preset(width=2048, vocab=32768, blocks=6, ff=None, experts=0, top=2) -> dict:
    """A layer stack of realistic sizes for benchmarks: per block one generalized-delta layer and one latent-attention layer; the
    feed-forward is dense, or table-routed experts of the same active size when `experts` > 0."""
    ff = ff or 4 * width
    heads = max(width // 128, 1)
    layers = []
    for _ in range(blocks):
        mlp_a = punilix_dense_mlp(ff)
        mlp_b = punilix_moe_mlp(ff // top, experts, top) if experts else punilix_dense_mlp(ff)
        layers.append(punilix_delta_layer(heads, 128, mlp_a))
        layers.append(punilix_latent_layer(heads, 128, 64, 128, 512, min(1536, width), mlp_b, base=10000.0,
                                           scaling={"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}))
    return punilix_config(width, vocab, layers, norm_groups=1, eps=1e-6, logit_softcap=30.0)


# ---------------------------------------------------------------------------------------------
# Gamanex (parallel-block family with two norms per layer, sigmoid attention, gated sublayers): config.json {"architecture": "Gamanex",
# "width", "vocab", "norm": {"eps"}, "logit_scale", "layers": [{"type": "attention", "mixer", "mlp"}]}; tensors embed, head, final.norm,
# l<i>.norm1/2, l<i>.mix.*, l<i>.mlp.*, l<i>.ls1/2, l<i>.rg1/2(.b)
# ---------------------------------------------------------------------------------------------
def gamanex_attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, mlp: dict | None, scale: float | None = None,
                            q_temp: tuple | None = None, kv_from: int | None = None) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
    if q_temp is not None:
        mixer["q_temp"] = {"coef": float(q_temp[0]), "every": int(q_temp[1])}
    if kv_from is not None:
        mixer["kv_from"] = int(kv_from)
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def gamanex_dense_mlp(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def gamanex_moe_mlp(ff: int, experts: int, top: int) -> dict:
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def gamanex_config(width: int, vocab: int, layers: list, eps: float = 1e-6, logit_scale: float = 1.0) -> dict:
    return {"architecture": "Gamanex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def gamanex_tensors(config: dict, seed: int = 0) -> dict:
    """Seeded random tensors of a Gamanex config: f32 values that bf16 holds exactly."""
    rng = np.random.default_rng(seed)
    W, V = config["width"], config["vocab"]

    def bf(x):
        return st_bits_to_f32(f32_to_bf16_bits(np.asarray(x, np.float32)))

    def mat(rows, cols, gain=1.0):
        return bf(rng.standard_normal((rows, cols), dtype=np.float32) * (gain / np.sqrt(cols)))

    def vec(n, mean=1.0, spread=0.1):
        return bf(mean + spread * rng.standard_normal(n, dtype=np.float32))

    t = {"embed": mat(V, W, np.sqrt(W)), "head": mat(V, W, 2.0), "final.norm": vec(W)}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = vec(W)
        t[p + "mix.q"], t[p + "mix.q.norm"] = mat(H * D, W), vec(H * D, 1.0, 0.2)
        if m.get("kv_from") is None:
            t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.k.norm"] = mat(G * D, W), mat(G * Dv, W), vec(G * D, 1.0, 0.2)
        t[p + "mix.r1"] = bf(np.abs(vec(H, 0.5, 0.3)) + 0.05)
        t[p + "mix.r2"] = bf(np.abs(vec(H, 0.3, 0.2)) + 0.05)
        t[p + "mix.pb"] = vec(H, -1.0, 0.5)
        t[p + "mix.o"] = mat(W, H * Dv)
        t[p + "ls1"], t[p + "rg1"], t[p + "rg1.b"] = vec(W, 0.7, 0.2), mat(W, W), vec(W, 0.3, 0.5)
        ml = L.get("mlp")
        if ml is None:
            continue
        t[p + "norm2"] = vec(W)
        t[p + "ls2"], t[p + "rg2"], t[p + "rg2.b"] = vec(W, 0.7, 0.2), mat(W, W), vec(W, 0.3, 0.5)
        if ml["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(ml["ff"], W, 1.5), mat(W, ml["ff"])
        else:
            f, E = ml["expert"]["ff"], ml["router"]["experts"]
            t[p + "mlp.router"], t[p + "mlp.router.b"] = mat(E, W, 2.0), vec(E, 0.0, 0.5)
            for x in range(E):
                q = f"{p}mlp.e{x}."
                t[q + "gate"], t[q + "up"], t[q + "down"] = mat(f, W, 1.5), mat(f, W, 1.5), mat(W, f)
    return t


def write_gamanex_model(config: dict, path, seed: int = 0, tensors: dict | None = None) -> Path:
    """config.json + model.safetensors (bf16). `tensors` overrides the seeded random ones (values are rounded to bf16)."""
    return write_punilix_model(config, path, seed, tensors if tensors is not None else gamanex_tensors(config, seed))


def gamanex_preset(width=2048, vocab=32768, blocks=6, ff=None, experts=0, top=2, kv_heads=None) -> dict:
    """A layer stack of realistic sizes for benchmarks: per block one attention layer that keeps its keys and values and one that
    borrows them; the feed-forward is dense, or (second layer of a block) routed experts of the same active size when `experts` > 0."""
    ff = ff or 4 * width
    heads = max(width // 128, 1)
    kv = kv_heads or heads
    layers = []
    for b in range(blocks):
        mlp_b = gamanex_moe_mlp(ff // top, experts, top) if experts else gamanex_dense_mlp(ff)
        layers.append(gamanex_attention_layer(heads, kv, 128, 128, gamanex_dense_mlp(ff), q_temp=(0.2, 128)))
        layers.append(gamanex_attention_layer(heads, kv, 128, 128, mlp_b, q_temp=(0.2, 128), kv_from=2 * b))
    return gamanex_config(width, vocab, layers, eps=1e-5, logit_scale=0.5)


# ---------------------------------------------------------------------------------------------
# Vugipel (sequential pre-norm sublayers; minGRU, or window attention + retention side by side; sigmoid-routed experts weighted on their
# input): config.json {"architecture": "Vugipel", "width", "vocab", "norm": {"eps"}, "layers": [{"type": "mingru" | "parallel", "mixer",
# "mlp"}]}; tensors embed, head, final.norm, l<i>.norm1/2 (stored around zero), l<i>.mix.*, l<i>.mlp.*
# ---------------------------------------------------------------------------------------------
def vugipel_mingru_layer(width: int, mlp: dict | None) -> dict:
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def vugipel_parallel_layer(heads: int, kv_heads: int, dim: int, vdim: int, window: int, keep_first: int, r_heads: int, r_dim: int, r_vdim: int,
                           mlp: dict | None, rot_dims: int | None = None, rot_base: float = 10000.0, scale: float | None = None,
                           softcap: float = 30.0, decay: list | None = None, left_scale: float = 1.0, right_scale: float = 1.0) -> dict:
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5),
            "softcap": float(softcap), "rot": {"base": float(rot_base), "dims": int(rot_dims if rot_dims is not None else dim)},
            "mask": {"size": int(window), "keep_first": int(keep_first)}}
    if decay is None:
        decay = [1.0 - 1.0 / (24.0 * (h % 8 + 1)) for h in range(r_heads)]
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": [float(d) for d in decay]}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": float(left_scale), "right": right, "right_scale": float(right_scale)}, "mlp": mlp}


def vugipel_moe_mlp(ff: int, experts: int, top: int) -> dict:
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def vugipel_config(width: int, vocab: int, layers: list, eps: float = 1e-6) -> dict:
    return {"architecture": "Vugipel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def vugipel_tensors(config: dict, seed: int = 0) -> dict:
    """Seeded random tensors of a Vugipel config: f32 values that bf16 holds exactly."""
    rng = np.random.default_rng(seed)
    W, V = config["width"], config["vocab"]

    def bf(x):
        return st_bits_to_f32(f32_to_bf16_bits(np.asarray(x, np.float32)))

    def mat(rows, cols, gain=1.0):
        return bf(rng.standard_normal((rows, cols), dtype=np.float32) * (gain / np.sqrt(cols)))

    def vec(n, mean=0.0, spread=0.1):
        return bf(mean + spread * rng.standard_normal(n, dtype=np.float32))

    t = {"embed": mat(V, W, np.sqrt(W)), "head": mat(V, W, 2.0), "final.norm": vec(W)}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        t[p + "norm1"] = vec(W)
        if L["type"] == "mingru":
            n = m["width"]
            t[p + "mix.z"], t[p + "mix.z.b"] = mat(n, W, 1.5), vec(n, 0.0, 0.5)
            t[p + "mix.x"], t[p + "mix.x.b"] = mat(n, W, 1.5), vec(n, 0.0, 0.5)
            t[p + "mix.g"], t[p + "mix.o"] = mat(n, W, 1.5), mat(W, n)
        else:
            A, R = m["left"], m["right"]
            H, G, D, Dv = A["heads"], A["kv_heads"], A["dim"], A["vdim"]
            l, r = p + "mix.left.", p + "mix.right."
            t[l + "q"], t[l + "q.b"] = mat(H * D, W), vec(H * D, 0.0, 0.2)
            t[l + "k"], t[l + "k.b"] = mat(G * D, W), vec(G * D, 0.0, 0.2)
            t[l + "v"], t[l + "v.b"] = mat(G * Dv, W), vec(G * Dv, 0.0, 0.2)
            t[l + "q.norm"], t[l + "k.norm"] = vec(D, 1.0, 0.2), vec(D, 1.0, 0.2)
            t[l + "temp"] = bf(np.abs(vec(H, 1.0, 0.3)) + 0.25)
            t[l + "o"], t[l + "o.b"] = mat(W, H * Dv), vec(W, 0.0, 0.1)
            Hr, Dr, Dvr = R["heads"], R["dim"], R["vdim"]
            t[r + "q"], t[r + "k"], t[r + "v"] = mat(Hr * Dr, W), mat(Hr * Dr, W), mat(Hr * Dvr, W)
            t[r + "g"], t[r + "o"] = mat(Hr * Dvr, W, 1.5), mat(W, Hr * Dvr)
        ml = L.get("mlp")
        if ml is None:
            continue
        t[p + "norm2"] = vec(W)
        f, E = ml["expert"]["ff"], ml["router"]["experts"]
        t[p + "mlp.router"] = mat(E, W, 2.0)
        for x in range(E):
            q = f"{p}mlp.e{x}."
            t[q + "gate"], t[q + "up"], t[q + "down"] = mat(f, W, 1.5), mat(f, W, 1.5), mat(W, f)
    return t


def write_vugipel_model(config: dict, path, seed: int = 0, tensors: dict | None = None) -> Path:
    """config.json + model.safetensors (bf16). `tensors` overrides the seeded random ones (values are rounded to bf16)."""
    return write_punilix_model(config, path, seed, tensors if tensors is not None else vugipel_tensors(config, seed))


def vugipel_preset(width=2048, vocab=32768, blocks=6, ff=None, experts=8, top=2, window=1024, keep_first=4) -> dict:
    """A layer stack of realistic sizes for benchmarks: per block one minGRU layer whose feed-forward is a single expert of size `ff` (the
    design's dense feed-forward) and one layer with window attention and retention side by side with `top` of `experts` routed experts of
    the same active size."""
    ff = ff or 4 * width
    heads = max(width // 128, 1)
    layers = []
    for _ in range(blocks):
        layers.append(vugipel_mingru_layer(width, vugipel_moe_mlp(ff, 1, 1)))
        layers.append(vugipel_parallel_layer(heads, max(heads // 4, 1), 128, 128, window, keep_first, max(heads // 2, 1), 128, 128,
                                             vugipel_moe_mlp(ff // top, experts, top), softcap=30.0, left_scale=0.8, right_scale=1.1))
    return vugipel_config(width, vocab, layers, eps=1e-5)


# ---- Vakesun: sandwich layers with Dynamic Tanh norms; attention, matrix memory (mLSTM) and windowed latent attention mixers ----------------

def vakesun_attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, mlp: dict | None, scale: float | None = None, rot_dims: int | None = None,
                            rot_base: float = 10000.0, scaling: dict | None = None) -> dict:
    rot_dims = dim if rot_dims is None else rot_dims
    rot = {"base": rot_base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if rot_dims:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def vakesun_mlstm_layer(heads: int, dim: int, vdim: int, mlp: dict | None, gate_cap: float = 15.0) -> dict:
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}, "mlp": mlp}


def vakesun_latent_layer(heads: int, dim: int, vdim: int, kv_rank: int, q_rank: int, window: int, mlp: dict | None, scale: float | None = None,
                         kv_from: int | None = None) -> dict:
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window},
             "scale": dim ** -0.5 if scale is None else scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def vakesun_dense_mlp(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def vakesun_config(width: int, vocab: int, layers: list, eps: float = 1e-6, residual_mult: float = 0.5, embedding_scale: float = 1.0,
                   side_dim: int = 8) -> dict:
    return {"architecture": "Vakesun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": residual_mult,
            "embedding": {"scale": embedding_scale}, "token_side": {"dim": side_dim}, "layers": layers}


def vakesun_tensors(config: dict, seed: int = 0) -> dict:
    """Seeded random tensors of a Vakesun config: f32 values that bf16 holds exactly."""
    rng = np.random.default_rng(seed)
    W, V = config["width"], config["vocab"]
    sd = config["token_side"]["dim"] if config.get("token_side") else 0
    nl = len(config["layers"])

    def bf(x):
        return st_bits_to_f32(f32_to_bf16_bits(np.asarray(x, np.float32)))

    def mat(rows, cols, gain=1.0):
        return bf(rng.standard_normal((rows, cols), dtype=np.float32) * (gain / np.sqrt(cols)))

    def vec(n, mean=0.0, spread=0.1):
        return bf(mean + spread * rng.standard_normal(n, dtype=np.float32))

    t = {"embed": mat(V, W, np.sqrt(W))}

    def dyt(name, alpha):
        t[name], t[name + ".b"] = vec(W, 1.0, 0.2), vec(W, 0.0, 0.1)
        t[name + ".alpha"] = bf(np.float32(alpha * (1.0 + 0.2 * rng.standard_normal()))).reshape(())      # a scalar

    dyt("final.norm", 0.6)
    if sd:
        t["side.embed"] = mat(V, nl * sd, np.sqrt(nl * sd))
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        dyt(p + "norm1", 0.7)
        dyt(p + "norm1b", 1.0)
        if L["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * D, W, 1.5), mat(G * D, W, 1.5), mat(G * Dv, W)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = vec(D, 1.0, 0.2), vec(D, 1.0, 0.2)
            t[p + "mix.o"] = mat(W, H * Dv)
        elif L["type"] == "mlstm":
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = mat(H * D, W, 1.5), mat(H * D, W, 1.5), mat(H * Dv, W), mat(H * Dv, W, 1.5)
            t[p + "mix.i"], t[p + "mix.i.b"] = mat(H, W, 2.0), vec(H, 0.0, 1.0)
            t[p + "mix.f"], t[p + "mix.f.b"] = mat(H, W, 2.0), vec(H, 3.0, 1.0)
            t[p + "mix.norm"], t[p + "mix.o"] = vec(H * Dv, 1.0, 0.2), mat(W, H * Dv)
        else:
            H, D, Dv, R, Q = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = mat(Q, W), vec(Q, 1.0, 0.2), mat(H * D, Q, 1.5)
            if m.get("kv_from") is None:
                t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(R, W), vec(R, 1.0, 0.2)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * D, R, 1.5), mat(H * Dv, R)
            t[p + "mix.sink"], t[p + "mix.g"] = vec(H, 0.5, 1.0), mat(H, W, 2.0)
            t[p + "mix.o"] = mat(W, H * Dv)
        if L.get("mlp") is not None:
            f = L["mlp"]["ff"]
            dyt(p + "norm2", 0.7)
            dyt(p + "norm2b", 1.0)
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(f, W, 1.5), mat(W, f)
        if sd:
            t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"] = mat(sd, W, 1.5), mat(W, sd), vec(W, 1.0, 0.2)
    return t


def write_vakesun_model(config: dict, path, seed: int = 0, tensors: dict | None = None) -> Path:
    """config.json + model.safetensors (bf16). `tensors` overrides the seeded random ones (values are rounded to bf16)."""
    return write_punilix_model(config, path, seed, tensors if tensors is not None else vakesun_tensors(config, seed))


def vakesun_preset(width=2048, vocab=32768, layers=8, ff=None, window=512, side_dim=256, memory_ff=True) -> dict:
    """A layer stack of realistic sizes for benchmarks, `layers` layers in the order: a windowed latent-attention layer, a full attention
    layer with grouped key / value heads, a matrix-memory layer (with a feed-forward only when memory_ff), a second latent-attention layer
    that reads the first one's latents; then again."""
    ff = ff or 4 * width
    heads = max(width // 128, 1)
    yarn = {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    out = []
    for i in range(layers):
        kind = i % 4
        if kind == 0:
            out.append(vakesun_latent_layer(heads, 128, 128, 512, min(1536, width), window, vakesun_dense_mlp(ff)))
        elif kind == 1:
            out.append(vakesun_attention_layer(heads, max(heads // 4, 1), 128, 128, vakesun_dense_mlp(ff), rot_dims=64, rot_base=1e6, scaling=yarn))
        elif kind == 2:
            out.append(vakesun_mlstm_layer(heads, 128, 128, vakesun_dense_mlp(ff) if memory_ff else None))
        else:
            out.append(vakesun_latent_layer(heads, 128, 128, 512, min(1536, width), window, vakesun_dense_mlp(ff), kv_from=i - 3))
    return vakesun_config(width, vocab, out, eps=1e-6, residual_mult=0.3, embedding_scale=1.0, side_dim=side_dim)
