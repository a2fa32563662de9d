"""Model configuration mirror of the reference's ``tensor.ModelConfig``.

Field meaning follows /root/reference purego/tensor/config.go:58-122; the
presets follow config.go:125-148 (GPT-2), :151-193 (Falcon), :330-376
(Granite-MoE, muP scalars from docs/ARCHITECTURE_GUIDE.md:1773-1776).  The
Llama-3.2 shapes are the HF config.json values the reference reads at load
(generic_loader.go:837-915); they are not in the reference tree.

``to_c()`` produces the ``nvllm_config`` struct of include/nvllm.h.
"""
from __future__ import annotations

import ctypes
import json
import os
from dataclasses import dataclass, replace
from typing import Optional, Tuple

ABI_VERSION = 1
KV_BLOCK_SIZE = 256  # nanovllm/sequence.go:52

ATTN_MHA, ATTN_GQA, ATTN_MQA = 0, 1, 2
NORM_LAYER, NORM_RMS = 0, 1
POS_LEARNED, POS_ROPE, POS_NONE = 0, 1, 2
ACT_GELU, ACT_SWIGLU = 0, 1
BLOCK_SEQUENTIAL, BLOCK_PARALLEL = 0, 1
PREC_FP32, PREC_BF16 = 0, 1
# enum nvllm_arch (checkpoint families of generic_loader.go:60-182)
ARCH_GPT2, ARCH_FALCON, ARCH_LLAMA, ARCH_GRANITE_MOE, ARCH_DUGOPEL, ARCH_ZOZONEX, ARCH_LAZOVIK, ARCH_SUTUVIK = 0, 1, 2, 3, 4, 5, 6, 7
MIXER_LATENT_ATTENTION, MIXER_WINDOW_ATTENTION, MIXER_DELTA, MIXER_GLA, MIXER_ATTN_TMIX = 1, 2, 3, 4, 5
MIXER_ATTENTION, MIXER_MAMBA2 = 6, 7
MLP_NONE, MLP_DENSE, MLP_MOE = 0, 1, 2
FFN_GLU_CLAMPED, FFN_RELU2, FFN_SWIGLU = 0, 1, 2
LBLOCK_PARALLEL_PRENORM, LBLOCK_SEQUENTIAL_POSTNORM, LBLOCK_SEQUENTIAL_PRENORM = 0, 1, 2
LPOS_NONE, LPOS_SINUSOIDAL = 0, 1
DT_F32, DT_BF16, DT_F16 = 0, 1, 2

# enum nvllm_weight_id
W_TOKEN_EMBEDDING, W_POS_EMBEDDING, W_FINAL_NORM_W, W_FINAL_NORM_B, W_LM_HEAD = 0, 1, 2, 3, 4
W_ATTN_NORM_W, W_ATTN_NORM_B, W_FFN_NORM_W, W_FFN_NORM_B = 16, 17, 18, 19
(W_MAMBA_IN_PROJ, W_MAMBA_CONV_W, W_MAMBA_CONV_B, W_MAMBA_DT_BIAS, W_MAMBA_A_LOG, W_MAMBA_D,
 W_MAMBA_NORM, W_MAMBA_OUT_PROJ) = 36, 37, 38, 39, 40, 41, 42, 43
W_Q, W_K, W_V, W_KV, W_O = 20, 21, 22, 23, 24
W_Q_BIAS, W_K_BIAS, W_V_BIAS, W_O_BIAS = 25, 26, 27, 28
W_FFN_W1, W_FFN_B1, W_FFN_W2, W_FFN_B2 = 29, 30, 31, 32
W_MOE_ROUTER, W_MOE_INPUT, W_MOE_OUTPUT = 33, 34, 35


class CConfig(ctypes.Structure):
    """``struct nvllm_config`` (include/nvllm.h)."""

    _fields_ = [
        ("abi_version", ctypes.c_int32),
        ("vocab_size", ctypes.c_int32),
        ("hidden", ctypes.c_int32),
        ("num_layers", ctypes.c_int32),
        ("num_heads", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("ffn_dim", ctypes.c_int32),
        ("max_seq_len", ctypes.c_int32),
        ("attention_type", ctypes.c_int32),
        ("norm_type", ctypes.c_int32),
        ("position_type", ctypes.c_int32),
        ("activation_type", ctypes.c_int32),
        ("block_style", ctypes.c_int32),
        ("tied_embedding", ctypes.c_int32),
        ("use_moe", ctypes.c_int32),
        ("num_experts", ctypes.c_int32),
        ("num_experts_per_tok", ctypes.c_int32),
        ("norm_eps", ctypes.c_float),
        ("embedding_multiplier", ctypes.c_float),
        ("attention_multiplier", ctypes.c_float),
        ("residual_multiplier", ctypes.c_float),
        ("logits_scaling", ctypes.c_float),
        ("rope_base", ctypes.c_double),
        ("precision", ctypes.c_int32),
        ("num_kv_blocks", ctypes.c_int32),
        ("max_num_seqs", ctypes.c_int32),
        ("max_batched_tokens", ctypes.c_int32),
        ("tp_size", ctypes.c_int32),
        ("tp_rank", ctypes.c_int32),
        ("device", ctypes.c_int32),
        ("mamba_num_heads", ctypes.c_int32),
        ("mamba_head_dim", ctypes.c_int32),
        ("mamba_state_size", ctypes.c_int32),
        ("mamba_n_groups", ctypes.c_int32),
        ("mamba_conv_kernel", ctypes.c_int32),
    ]


@dataclass(frozen=True)
class ModelConfig:
    name: str
    vocab_size: int
    hidden: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn_dim: int
    max_seq_len: int
    attention_type: int
    norm_type: int
    position_type: int
    activation_type: int
    block_style: int
    tied_embedding: bool
    norm_eps: float
    rope_base: float = 10000.0
    use_moe: bool = False
    num_experts: int = 0
    num_experts_per_tok: int = 0
    embedding_multiplier: float = 0.0
    attention_multiplier: float = 0.0
    residual_multiplier: float = 0.0
    logits_scaling: float = 0.0
    has_ffn_bias: bool = False  # GPT-2 c_fc/c_proj biases; optional at the boundary
    eos_token_id: int = -1
    # Granite-4 hybrid (purego/tensor/config.go:100-115): hybrid_layers[l] = True -> Mamba2 block
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    mamba_state_size: int = 0
    mamba_n_groups: int = 0
    mamba_conv_kernel: int = 0
    hybrid_layers: tuple = ()

    def is_mamba(self, layer: int) -> bool:
        return bool(self.hybrid_layers) and bool(self.hybrid_layers[layer])

    def mamba_dims(self):
        """(E = expand * hidden, conv_dim, in_proj rows)."""
        E = self.mamba_num_heads * self.mamba_head_dim
        conv = E + 2 * self.mamba_n_groups * self.mamba_state_size
        return E, conv, E + conv + self.mamba_num_heads

    def kv_heads(self) -> int:
        if self.attention_type == ATTN_MQA:
            return 1
        if self.attention_type == ATTN_MHA:
            return self.num_heads
        return self.num_kv_heads

    def matmul_params(self) -> int:
        """Parameters of every matmul touched once per decode step."""
        H, F, L = self.hidden, self.ffn_dim, self.num_layers
        q = self.num_heads * self.head_dim
        kv = self.kv_heads() * self.head_dim
        attn = H * q + 2 * H * kv + q * H
        if self.use_moe:
            ffn = H * self.num_experts + self.num_experts * (2 * F * H + H * F)
        elif self.activation_type == ACT_SWIGLU:
            ffn = 3 * H * F
        else:
            ffn = 2 * H * F
        return L * (attn + ffn) + H * self.vocab_size

    def kv_bytes_per_token(self, bytes_per_el: int = 2) -> int:
        return 2 * self.num_layers * self.kv_heads() * self.head_dim * bytes_per_el

    def to_c(self, precision: int, num_kv_blocks: int = -1, max_num_seqs: int = 512,
             max_batched_tokens: int = 16384, device: int = 0, tp_size: int = 1,
             tp_rank: int = 0) -> CConfig:
        c = CConfig()
        c.abi_version = ABI_VERSION
        c.vocab_size = self.vocab_size
        c.hidden = self.hidden
        c.num_layers = self.num_layers
        c.num_heads = self.num_heads
        c.num_kv_heads = self.kv_heads()
        c.head_dim = self.head_dim
        c.ffn_dim = self.ffn_dim
        c.max_seq_len = self.max_seq_len
        c.attention_type = self.attention_type
        c.norm_type = self.norm_type
        c.position_type = self.position_type
        c.activation_type = self.activation_type
        c.block_style = self.block_style
        c.tied_embedding = int(self.tied_embedding)
        c.use_moe = int(self.use_moe)
        c.num_experts = self.num_experts
        c.num_experts_per_tok = self.num_experts_per_tok
        c.norm_eps = self.norm_eps
        c.embedding_multiplier = self.embedding_multiplier
        c.attention_multiplier = self.attention_multiplier
        c.residual_multiplier = self.residual_multiplier
        c.logits_scaling = self.logits_scaling
        c.rope_base = self.rope_base
        c.precision = precision
        c.num_kv_blocks = num_kv_blocks
        c.max_num_seqs = max_num_seqs
        c.max_batched_tokens = max_batched_tokens
        c.tp_size = tp_size
        c.tp_rank = tp_rank
        c.device = device
        c.mamba_num_heads = self.mamba_num_heads
        c.mamba_head_dim = self.mamba_head_dim
        c.mamba_state_size = self.mamba_state_size
        c.mamba_n_groups = self.mamba_n_groups
        c.mamba_conv_kernel = self.mamba_conv_kernel
        return c


def gpt2_small() -> ModelConfig:  # config.go:125-148
    return ModelConfig("gpt2", 50257, 768, 12, 12, 12, 64, 3072, 1024, ATTN_MHA, NORM_LAYER,
                       POS_LEARNED, ACT_GELU, BLOCK_SEQUENTIAL, True, 1e-5, has_ffn_bias=True,
                       eos_token_id=50256)


def llama32_1b() -> ModelConfig:  # HF meta-llama/Llama-3.2-1B; ref MaxSeqLen preset 4096 (config.go:222)
    return ModelConfig("llama-3.2-1b", 128256, 2048, 16, 32, 8, 64, 8192, 4096, ATTN_GQA, NORM_RMS,
                       POS_ROPE, ACT_SWIGLU, BLOCK_SEQUENTIAL, True, 1e-5, rope_base=500000.0,
                       eos_token_id=128001)


def llama32_3b() -> ModelConfig:  # HF meta-llama/Llama-3.2-3B
    return ModelConfig("llama-3.2-3b", 128256, 3072, 28, 24, 8, 128, 8192, 4096, ATTN_GQA, NORM_RMS,
                       POS_ROPE, ACT_SWIGLU, BLOCK_SEQUENTIAL, True, 1e-5, rope_base=500000.0,
                       eos_token_id=128001)


def granite_moe_1b() -> ModelConfig:  # config.go:330-376 + docs/ARCHITECTURE_GUIDE.md:1773-1776
    return ModelConfig("granite-3.0-1b-a400m", 49155, 1024, 24, 16, 8, 64, 512, 4096, ATTN_GQA,
                       NORM_RMS, POS_ROPE, ACT_SWIGLU, BLOCK_SEQUENTIAL, True, 1e-6,
                       rope_base=10000.0, use_moe=True, num_experts=32, num_experts_per_tok=8,
                       embedding_multiplier=12.0, attention_multiplier=0.015625,
                       residual_multiplier=0.22, logits_scaling=6.0, eos_token_id=0)


def falcon_7b() -> ModelConfig:  # config.go:151-177
    return ModelConfig("falcon-7b", 65024, 4544, 32, 71, 1, 64, 18176, 2048, ATTN_MQA, NORM_LAYER,
                       POS_ROPE, ACT_GELU, BLOCK_PARALLEL, False, 1e-5, rope_base=10000.0,
                       eos_token_id=11)


def tiny(base: ModelConfig, **kw) -> ModelConfig:
    """Scaled-down sibling of a preset for parity tests the CPU oracle finishes in seconds."""
    return replace(base, name=base.name + "-tiny", **kw)


def tiny_gpt2(**kw) -> ModelConfig:
    d = dict(vocab_size=1000, hidden=128, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=32,
             ffn_dim=512, max_seq_len=640)
    d.update(kw)
    return tiny(gpt2_small(), **d)


def tiny_llama(**kw) -> ModelConfig:
    d = dict(vocab_size=1000, hidden=256, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=32,
             ffn_dim=512, max_seq_len=1024)
    d.update(kw)
    return tiny(llama32_1b(), **d)


def tiny_granite(**kw) -> ModelConfig:
    d = dict(vocab_size=1000, hidden=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
             ffn_dim=64, max_seq_len=1024, num_experts=8, num_experts_per_tok=2)
    d.update(kw)
    return tiny(granite_moe_1b(), **d)


def tiny_hybrid(**kw) -> ModelConfig:
    """Granite-4-style hybrid: Mamba2 and GQA attention blocks (no positional encoding,
    config.go:241-300), shared SwiGLU MLP, muP multipliers."""
    d = dict(vocab_size=1000, hidden=128, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=32,
             ffn_dim=256, max_seq_len=1024, position_type=POS_NONE, use_moe=False, num_experts=0,
             num_experts_per_tok=0, mamba_num_heads=8, mamba_head_dim=32, mamba_state_size=16,
             mamba_n_groups=2, mamba_conv_kernel=4, hybrid_layers=(True, False, True, True))
    d.update(kw)
    return replace(tiny(granite_moe_1b(), **d), name="granite-4-hybrid-tiny")


def tiny_falcon(**kw) -> ModelConfig:
    d = dict(vocab_size=1000, hidden=7 * 32, num_layers=2, num_heads=7, num_kv_heads=1, head_dim=32,
             ffn_dim=4 * 7 * 32, max_seq_len=1024)
    d.update(kw)
    return tiny(falcon_7b(), **d)


PRESETS = {
    "gpt2": gpt2_small,
    "llama-3.2-1b": llama32_1b,
    "llama-3.2-3b": llama32_3b,
    "granite-moe-1b": granite_moe_1b,
    "falcon-7b": falcon_7b,
}


# ---- models given as a list of layers (include/nvllm.h: nvllm_layer_spec) ----------------

class CLayerSpec(ctypes.Structure):
    """``struct nvllm_layer_spec``."""

    _fields_ = [
        ("mixer", ctypes.c_int32),
        ("heads", ctypes.c_int32), ("dim", ctypes.c_int32), ("rot_dim", ctypes.c_int32),
        ("vdim", ctypes.c_int32), ("kv_rank", ctypes.c_int32), ("q_rank", ctypes.c_int32),
        ("rot_dims", ctypes.c_int32), ("kv_from", ctypes.c_int32),
        ("rot_base", ctypes.c_float), ("scale", ctypes.c_float),
        ("mlp", ctypes.c_int32), ("ff", ctypes.c_int32), ("limit", ctypes.c_float),
        ("experts", ctypes.c_int32), ("top", ctypes.c_int32),
        ("groups", ctypes.c_int32), ("keep_groups", ctypes.c_int32),
        ("router_scale", ctypes.c_float),
        ("kv_heads", ctypes.c_int32), ("window", ctypes.c_int32), ("sink", ctypes.c_int32),
        ("qk_norm", ctypes.c_int32), ("conv", ctypes.c_int32), ("act", ctypes.c_int32),
        ("chunk", ctypes.c_int32), ("softcap", ctypes.c_float), ("proj_bias", ctypes.c_int32),
        ("out_gate", ctypes.c_int32),
        ("rot_factor", ctypes.c_float), ("rot_original", ctypes.c_float), ("rot_fast", ctypes.c_float),
        ("rot_slow", ctypes.c_float),
        ("tau", ctypes.c_float), ("lowrank", ctypes.c_int32), ("heads2", ctypes.c_int32), ("dim2", ctypes.c_int32),
        ("mix_scale", ctypes.c_float), ("mix2_scale", ctypes.c_float),
        ("route_sigmoid", ctypes.c_int32), ("weight_on_input", ctypes.c_int32), ("shared_ff", ctypes.c_int32),
        ("rot_pairs", ctypes.c_int32), ("rot_piecewise", ctypes.c_int32),
        ("qtemp_coef", ctypes.c_float), ("qtemp_every", ctypes.c_int32), ("head_temp", ctypes.c_int32),
        ("dist_slope", ctypes.c_float), ("sink_learned", ctypes.c_int32), ("v_mix", ctypes.c_int32),
        ("head_gate", ctypes.c_int32),
        ("state", ctypes.c_int32), ("ssm_groups", ctypes.c_int32), ("norm_groups", ctypes.c_int32),
        ("route_correction", ctypes.c_int32), ("group_top2", ctypes.c_int32), ("route_norm", ctypes.c_int32),
    ]


class CLayeredConfig(ctypes.Structure):
    """``struct nvllm_layered_config``."""

    _fields_ = [
        ("abi_version", ctypes.c_int32), ("vocab_size", ctypes.c_int32), ("hidden", ctypes.c_int32),
        ("num_layers", ctypes.c_int32), ("norm_eps", ctypes.c_float),
        ("embedding_scale", ctypes.c_float), ("logit_softcap", ctypes.c_float),
        ("precision", ctypes.c_int32), ("num_kv_blocks", ctypes.c_int32),
        ("max_num_seqs", ctypes.c_int32), ("max_batched_tokens", ctypes.c_int32),
        ("device", ctypes.c_int32),
        ("block_style", ctypes.c_int32), ("position", ctypes.c_int32), ("tied_head", ctypes.c_int32),
        ("norm_offset", ctypes.c_float), ("num_state_slots", ctypes.c_int32),
        ("loop_start", ctypes.c_int32), ("loop_stop", ctypes.c_int32), ("loop_times", ctypes.c_int32),
        ("norm_groups", ctypes.c_int32), ("embed_norm", ctypes.c_int32), ("mixer_conv", ctypes.c_int32),
        ("side_dim", ctypes.c_int32), ("logit_scale", ctypes.c_float),
    ]


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its mixer (latent attention, window attention or delta rule) and its
    feed-forward (none, dense, or MoE)."""
    heads: int
    dim: int
    vdim: int
    rot_dim: int = 0
    kv_rank: int = 0
    q_rank: int = 0
    rot_base: float = 0.0
    rot_dims: int = 0
    scale: float = 1.0
    kv_from: int = -1
    mixer: int = MIXER_LATENT_ATTENTION
    mlp: int = MLP_NONE
    ff: int = 0
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    groups: int = 0
    keep_groups: int = 0
    router_scale: float = 1.0
    kv_heads: int = 0
    window: int = 0
    sink: int = 0
    qk_norm: int = 0
    conv: int = 0
    act: int = FFN_GLU_CLAMPED
    chunk: int = 0
    softcap: float = 0.0
    proj_bias: int = 0
    out_gate: int = 0
    rot_factor: float = 0.0
    rot_original: float = 0.0
    rot_fast: float = 0.0
    rot_slow: float = 0.0
    tau: float = 0.0
    lowrank: int = 0
    heads2: int = 0
    dim2: int = 0
    mix_scale: float = 1.0
    mix2_scale: float = 1.0
    route_sigmoid: int = 0
    weight_on_input: int = 0
    shared_ff: int = 0
    rot_pairs: int = 0
    rot_piecewise: int = 0
    qtemp_coef: float = 0.0
    qtemp_every: int = 0
    head_temp: int = 0
    dist_slope: float = 0.0
    sink_learned: int = 0
    v_mix: int = 0
    head_gate: int = 0
    state: int = 0
    ssm_groups: int = 0
    norm_groups: int = 0
    route_correction: int = 0
    group_top2: int = 0
    route_norm: int = 0

    def to_c(self) -> CLayerSpec:
        c = CLayerSpec()
        for name, _ in CLayerSpec._fields_:
            setattr(c, name, getattr(self, name))
        return c

    def tensor_shapes(self, layer: int, width: int) -> dict:
        """Checkpoint names and shapes of this layer's tensors (linears [out, in])."""
        p = f"l{layer}."
        if self.mixer in (MIXER_GLA, MIXER_ATTN_TMIX):
            return self._prenorm_shapes(p, width)
        if self.mixer in (MIXER_ATTENTION, MIXER_MAMBA2):
            return self._prenorm2_shapes(p, width)
        if self.mixer == MIXER_WINDOW_ATTENTION:
            d = {p + "norm1": (width,), p + "mix.q": (self.heads * self.dim, width),
                 p + "mix.o": (width, self.heads * self.vdim)}
            if self.kv_from < 0:
                d[p + "mix.k"] = (self.kv_heads * self.dim, width)
                d[p + "mix.v"] = (self.kv_heads * self.vdim, width)
        elif self.mixer == MIXER_DELTA:
            qk, v = self.kv_heads * self.dim, self.heads * self.vdim
            d = {p + "norm1": (width,), p + "mix.q": (qk, width), p + "mix.k": (qk, width),
                 p + "mix.v": (v, width), p + "mix.q.conv": (qk, self.conv),
                 p + "mix.k.conv": (qk, self.conv), p + "mix.v.conv": (v, self.conv),
                 p + "mix.b": (self.heads, width), p + "mix.a": (self.heads, width),
                 p + "mix.A_log": (self.heads,), p + "mix.dt_bias": (self.heads,),
                 p + "mix.norm": (self.vdim,), p + "mix.g": (v, width), p + "mix.o": (width, v)}
        else:
            d = {p + "norm1": (width,),
                 p + "mix.dq": (self.q_rank, width), p + "mix.dq.norm": (self.q_rank,),
                 p + "mix.uq": (self.heads * (self.dim + self.rot_dim), self.q_rank),
                 p + "mix.uk": (self.heads * self.dim, self.kv_rank),
                 p + "mix.uv": (self.heads * self.vdim, self.kv_rank),
                 p + "mix.g": (self.heads, width), p + "mix.o": (width, self.heads * self.vdim)}
            if self.kv_from < 0:
                d[p + "mix.dkv"] = (self.kv_rank + self.rot_dim, width)
                d[p + "mix.dkv.norm"] = (self.kv_rank,)
        if self.mlp == MLP_DENSE and self.act == FFN_RELU2:
            d.update({p + "norm2": (width,), p + "mlp.up": (self.ff, width),
                      p + "mlp.down": (width, self.ff)})
        elif self.mlp == MLP_DENSE:
            d.update({p + "mlp.gate": (self.ff, width), p + "mlp.up": (self.ff, width),
                      p + "mlp.down": (width, self.ff)})
        elif self.mlp == MLP_MOE:
            d[p + "mlp.router"] = (self.experts, width)
            for e in range(self.experts):
                d.update({f"{p}mlp.e{e}.gate": (self.ff, width), f"{p}mlp.e{e}.up": (self.ff, width),
                          f"{p}mlp.e{e}.down": (width, self.ff)})
        return d


def _prenorm_shapes(self, p: str, width: int) -> dict:
    hd, hv = self.heads * self.dim, self.heads * self.vdim
    d = {p + "norm1": (width,)}
    if self.mixer == MIXER_GLA:
        d.update({p + "mix.q": (hd, width), p + "mix.k": (hd, width), p + "mix.v": (hv, width),
                  p + "mix.g": (hv, width), p + "mix.o": (width, hv), p + "mix.norm": (self.vdim,),
                  p + "mix.a1": (self.lowrank, width), p + "mix.a2": (hd, self.lowrank), p + "mix.a2.b": (hd,)})
    else:
        m = p + "mix.left."
        nk, nv = self.kv_heads * self.dim, self.kv_heads * self.vdim
        d.update({m + "q": (hd, width), m + "k": (nk, width), m + "v": (nv, width),
                  m + "q.norm": (hd,), m + "k.norm": (nk,), m + "q.conv": (hd, self.conv),
                  m + "k.conv": (nk, self.conv), m + "v.conv": (nv, self.conv), m + "o": (width, hv)})
        if self.proj_bias:
            d.update({m + "q.b": (hd,), m + "k.b": (nk,), m + "v.b": (nv,), m + "o.b": (width,)})
        if self.out_gate:
            d[m + "g"] = (hv, width)
        m = p + "mix.right."
        hd2 = self.heads2 * self.dim2
        d.update({m + "mu." + x: (width,) for x in "rkvgw"})
        d.update({m + "r": (hd2, width), m + "k": (hd2, width), m + "v": (hd2, width), m + "g": (hd2, width),
                  m + "w1": (self.lowrank, width), m + "w2": (hd2, self.lowrank), m + "w0": (hd2,),
                  m + "u": (self.heads2, self.dim2), m + "norm": (hd2,), m + "o": (width, hd2)})
    if self.mlp == MLP_MOE:
        d[p + "norm2"] = (width,)
        d[p + "mlp.router"] = (self.experts, width)
        for e in range(self.experts):
            d.update({f"{p}mlp.e{e}.up": (self.ff, width), f"{p}mlp.e{e}.down": (width, self.ff)})
        if self.shared_ff > 0:
            d.update({p + "mlp.shared.up": (self.shared_ff, width), p + "mlp.shared.down": (width, self.shared_ff),
                      p + "mlp.shared.sg": (1, width)})
    return d


LayerSpec._prenorm_shapes = _prenorm_shapes


def _prenorm2_shapes(self, p: str, width: int) -> dict:
    """Attention with its options / Mamba-2, and the mixture of gated experts."""
    d = {p + "norm1": (width,)}
    m = p + "mix."
    if self.mixer == MIXER_ATTENTION:
        hv = self.heads * self.vdim
        d.update({m + "q": (self.heads * self.dim, width), m + "k": (self.kv_heads * self.dim, width),
                  m + "v": (self.kv_heads * self.vdim, width), m + "o": (width, hv)})
        if self.qk_norm == 3:
            d.update({m + "q.norm": (self.dim,), m + "k.norm": (self.dim,)})
        if self.v_mix:
            d[m + "vmix"] = ()
        if self.sink_learned:
            d[m + "sink"] = (self.heads,)
        if self.head_temp:
            d[m + "temp"] = (self.heads,)
        if self.head_gate:
            d[m + "g"] = (self.heads, width)
    else:
        inner, gn = self.heads * self.vdim, self.ssm_groups * self.state
        d.update({m + "in": (2 * inner + 2 * gn + self.heads, width), m + "conv": (inner + 2 * gn, self.conv),
                  m + "conv.b": (inner + 2 * gn,), m + "dt_bias": (self.heads,), m + "A_log": (self.heads,),
                  m + "D": (self.heads,), m + "norm": (inner,), m + "o": (width, inner)})
    if self.mlp == MLP_MOE:
        d[p + "norm2"] = (width,)
        d[p + "mlp.router"] = (self.experts, width)
        if self.route_correction:
            d[p + "mlp.correction"] = (self.experts,)
        for e in range(self.experts):
            d.update({f"{p}mlp.e{e}.gate": (self.ff, width), f"{p}mlp.e{e}.up": (self.ff, width),
                      f"{p}mlp.e{e}.down": (width, self.ff)})
    return d


LayerSpec._prenorm2_shapes = _prenorm2_shapes


@dataclass(frozen=True)
class ListedModelConfig:
    """A model whose config.json lists its layers (architectures "Dugopel", "Zozonex", "Lazovik", "Sutuvik")."""
    name: str
    vocab_size: int
    hidden: int
    layers: Tuple[LayerSpec, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    eos_token_id: int = -1
    arch: int = ARCH_DUGOPEL
    block_style: int = LBLOCK_PARALLEL_PRENORM
    position: int = LPOS_NONE
    tied_head: bool = False
    norm_offset: float = 0.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0   # >= 1 with loop_stop > loop_start: layers [start, stop) run that often in a row
    norm_groups: int = 0  # > 1: the stream's norms work on that many equal parts of the row
    embed_norm: bool = False
    mixer_conv: int = 0   # taps of the causal convolution added to what every mixer reads
    side_dim: int = 0     # entries of the per-layer token input
    logit_scale: float = 0.0

    @property
    def has_loop(self) -> bool:
        return self.loop_times >= 1 and self.loop_stop > self.loop_start

    @property
    def runs(self) -> Tuple[int, ...]:
        """Layer indices in execution order (a repeated run of layers counts every pass)."""
        n = len(self.layers)
        if not self.has_loop:
            return tuple(range(n))
        return tuple(range(self.loop_start)) + tuple(range(self.loop_start, self.loop_stop)) * self.loop_times + \
            tuple(range(self.loop_stop, n))

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @property
    def needs_state_slots(self) -> bool:
        """True when some layer keeps recurrent state per sequence (delta rule)."""
        return self.mixer_conv > 1 or any(l.mixer in (MIXER_DELTA, MIXER_GLA, MIXER_ATTN_TMIX, MIXER_MAMBA2)
                                          for l in self.layers)

    def tensor_shapes(self) -> dict:
        d = {"embed": (self.vocab_size, self.hidden), "final.norm": (self.hidden,)}
        if not self.tied_head:
            d["head"] = (self.vocab_size, self.hidden)
        if self.has_loop:
            d["loop.step"] = (self.loop_times, self.hidden)
        if self.embed_norm:
            d["embed.norm"] = (self.hidden,)
        if self.side_dim > 0:
            d["side.embed"] = (self.vocab_size, len(self.layers) * self.side_dim)
        for i, l in enumerate(self.layers):
            d.update(l.tensor_shapes(i, self.hidden))
            if self.mixer_conv > 1:
                d[f"l{i}.canon1"] = (self.hidden, self.mixer_conv)
            if self.side_dim > 0:
                d.update({f"l{i}.side.gate": (self.side_dim, self.hidden), f"l{i}.side.proj": (self.hidden, self.side_dim),
                          f"l{i}.side.norm": (self.hidden,)})
        return d

    def matmul_params(self) -> int:
        shapes = self.tensor_shapes()
        n = sum(s[0] * s[1] for k, s in shapes.items()
                if len(s) == 2 and not k.endswith(".conv") and not k.endswith(".canon1") and k != "side.embed")
        return n - (0 if self.tied_head else self.vocab_size * self.hidden)

    def cache_bytes_per_token(self, bytes_per_el: int = 2) -> int:
        n = 0
        for l in (self.layers[i] for i in self.runs):
            if l.mixer in (MIXER_ATTN_TMIX, MIXER_ATTENTION):
                n += l.kv_heads * (l.dim + l.vdim) * bytes_per_el
            elif l.mixer == MIXER_LATENT_ATTENTION and l.kv_from < 0:
                n += (l.kv_rank + l.rot_dim) * bytes_per_el
            elif l.mixer == MIXER_WINDOW_ATTENTION and l.kv_from < 0:
                n += l.kv_heads * (l.dim + l.vdim) * bytes_per_el
        return n

    def state_bytes_per_sequence(self) -> int:
        """fp32 recurrent state + convolution tail of the delta-rule layers."""
        n = sum(4 * (l.heads * l.dim * l.vdim + (l.conv - 1) * (2 * l.kv_heads * l.dim + l.heads * l.vdim))
                for l in self.layers if l.mixer == MIXER_DELTA)
        for l in (self.layers[i] for i in self.runs):
            if l.mixer == MIXER_GLA:
                n += 4 * l.heads * l.dim * l.vdim
            elif l.mixer == MIXER_ATTN_TMIX:
                n += 4 * (l.heads2 * l.dim2 * l.dim2 + self.hidden +
                          (l.conv - 1) * (l.heads * l.dim + l.kv_heads * (l.dim + l.vdim)))
            elif l.mixer == MIXER_MAMBA2:
                n += 4 * (l.heads * l.state * l.vdim + (l.conv - 1) * (l.heads * l.vdim + 2 * l.ssm_groups * l.state))
            if self.mixer_conv > 1:
                n += 4 * (self.mixer_conv - 1) * self.hidden
        return n

    def to_c(self, precision: int, num_kv_blocks: int = -1, max_num_seqs: int = 512,
             max_batched_tokens: int = 16384, device: int = 0, num_state_slots: int = 0):
        c = CLayeredConfig()
        c.abi_version = ABI_VERSION
        c.vocab_size, c.hidden, c.num_layers = self.vocab_size, self.hidden, len(self.layers)
        c.norm_eps, c.embedding_scale, c.logit_softcap = self.norm_eps, self.embedding_scale, self.logit_softcap
        c.precision, c.num_kv_blocks = precision, num_kv_blocks
        c.max_num_seqs, c.max_batched_tokens, c.device = max_num_seqs, max_batched_tokens, device
        c.block_style, c.position, c.tied_head = self.block_style, self.position, int(self.tied_head)
        c.norm_offset, c.num_state_slots = self.norm_offset, num_state_slots
        c.loop_start, c.loop_stop, c.loop_times = self.loop_start, self.loop_stop, self.loop_times
        c.norm_groups, c.embed_norm, c.mixer_conv = self.norm_groups, int(self.embed_norm), self.mixer_conv
        c.side_dim, c.logit_scale = self.side_dim, self.logit_scale
        specs = (CLayerSpec * len(self.layers))(*[l.to_c() for l in self.layers])
        return c, specs


def _dugopel_layer(i: int, lc: dict) -> LayerSpec:
    if lc.get("type") != "latent_attention":
        raise ValueError(f"layer {i}: unknown layer type {lc.get('type')!r}")
    m = lc["mixer"]
    kw = dict(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
              kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), rot_base=float(m["rot"]["base"]),
              rot_dims=int(m["rot"]["dims"]), scale=float(m["scale"]),
              kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else -1)
    mlp = lc.get("mlp")
    if mlp is None:
        pass
    elif mlp["kind"] == "dense":
        kw.update(mlp=MLP_DENSE, ff=int(mlp["ff"]), limit=float(mlp["limit"]))
    elif mlp["kind"] == "moe":
        r = mlp["router"]
        g = r.get("groups") or {}
        kw.update(mlp=MLP_MOE, ff=int(mlp["expert"]["ff"]), limit=float(mlp["expert"]["limit"]),
                  experts=int(r["experts"]), top=int(r["top"]), groups=int(g.get("count", 0)),
                  keep_groups=int(g.get("keep", 0)), router_scale=float(r.get("scale", 1.0)))
    else:
        raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
    return LayerSpec(**kw)


def dugopel_from_json(j: dict) -> ListedModelConfig:
    """config.json of the Dugopel design: every size and constant comes from the file."""
    return ListedModelConfig(
        name="dugopel", vocab_size=int(j["vocab"]), hidden=int(j["width"]),
        layers=tuple(_dugopel_layer(i, lc) for i, lc in enumerate(j["layers"])),
        norm_eps=float(j["norm"]["eps"]), embedding_scale=float(j["embedding"]["scale"]),
        logit_softcap=float(j.get("logit_softcap") or 0.0))


def _zozonex_layer(i: int, lc: dict) -> LayerSpec:
    m = lc["mixer"]
    kind = lc.get("type")
    kw = dict(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]))
    if kind == "delta":
        kw.update(mixer=MIXER_DELTA, conv=int(m["conv"]))
    elif kind == "attention":
        kw.update(mixer=MIXER_WINDOW_ATTENTION, scale=float(m["scale"]), window=int(m["mask"]["size"]),
                  sink=1, qk_norm=1, kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else -1)
    else:
        raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    mlp = lc.get("mlp")
    if mlp is None:
        pass
    elif mlp["kind"] == "dense":
        kw.update(mlp=MLP_DENSE, ff=int(mlp["ff"]), act=FFN_RELU2)
    else:
        raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
    return LayerSpec(**kw)


def zozonex_from_json(j: dict) -> ListedModelConfig:
    """config.json of the Zozonex design: delta-rule and sliding-window attention layers, each
    sublayer followed by an RMS norm whose weight is stored around zero, sinusoidal positions
    added to the scaled embedding, logits through the embedding table."""
    return ListedModelConfig(
        name="zozonex", vocab_size=int(j["vocab"]), hidden=int(j["width"]),
        layers=tuple(_zozonex_layer(i, lc) for i, lc in enumerate(j["layers"])),
        norm_eps=float(j["norm"]["eps"]), embedding_scale=float(j["embedding"]["scale"]),
        arch=ARCH_ZOZONEX, block_style=LBLOCK_SEQUENTIAL_POSTNORM, position=LPOS_SINUSOIDAL,
        tied_head=True, norm_offset=1.0)


def _lazovik_layer(i: int, lc: dict, shapes: dict) -> LayerSpec:
    m = lc["mixer"]
    kind = lc.get("type")

    def inner(name: str) -> int:
        # the inner size of the decay's two-step projection is given by the tensor's shape only
        if name not in shapes:
            raise ValueError(f"layer {i}: the checkpoint has no tensor {name}")
        return int(shapes[name][0])

    if kind == "gla":
        kw = dict(mixer=MIXER_GLA, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                  tau=float(m["tau"]), lowrank=inner(f"l{i}.mix.a1"))
    elif kind == "parallel":
        a, b = m["left"], m["right"]
        rot = a.get("rot") or {}
        sc = rot.get("scaling") or {}
        mask = a.get("mask") or {}
        kw = dict(mixer=MIXER_ATTN_TMIX, heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]),
                  vdim=int(a["vdim"]), conv=int(a.get("conv") or 1), scale=float(a["scale"]),
                  softcap=float(a.get("softcap") or 0.0), chunk=int(mask.get("size") or 0), qk_norm=2,
                  proj_bias=1, out_gate=1, rot_dims=int(rot.get("dims") or 0), rot_base=float(rot.get("base") or 0.0),
                  rot_factor=float(sc.get("factor") or 0.0), rot_original=float(sc.get("original") or 0.0),
                  rot_fast=float(sc.get("fast") or 0.0), rot_slow=float(sc.get("slow") or 0.0),
                  heads2=int(b["heads"]), dim2=int(b["dim"]), lowrank=inner(f"l{i}.mix.right.w1"),
                  mix_scale=float(m["left_scale"]), mix2_scale=float(m["right_scale"]))
    else:
        raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    mlp = lc.get("mlp")
    if mlp is None:
        pass
    elif mlp["kind"] == "moe":
        r = mlp["router"]
        kw.update(mlp=MLP_MOE, act=FFN_RELU2, ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]),
                  route_sigmoid=1, weight_on_input=1, shared_ff=int((mlp.get("shared") or {}).get("ff") or 0))
    else:
        raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
    return LayerSpec(**kw)


def lazovik_from_json(j: dict, shapes: Optional[dict] = None) -> ListedModelConfig:
    """config.json of the Lazovik design: gated-linear-attention layers and layers that run a
    convolved, gated, chunk-masked attention beside RWKV-style time mixing; pre-norm blocks, a
    mixture of squared-ReLU experts with an always-on expert; a run of layers may repeat.
    `shapes`: tensor name -> shape of the checkpoint (sizes that only a tensor's shape gives)."""
    lp = j.get("loop") or {}
    times = int(lp.get("times") or 0)  # a run that "repeats" once still opens its pass with the pass's vector
    return ListedModelConfig(
        name="lazovik", vocab_size=int(j["vocab"]), hidden=int(j["width"]),
        layers=tuple(_lazovik_layer(i, lc, shapes or {}) for i, lc in enumerate(j["layers"])),
        norm_eps=float(j["norm"]["eps"]), arch=ARCH_LAZOVIK, block_style=LBLOCK_SEQUENTIAL_PRENORM,
        loop_start=int(lp.get("start") or 0) if times >= 1 else 0,
        loop_stop=int(lp.get("stop") or 0) if times >= 1 else 0, loop_times=times)


# the distance bias of Sutuvik's first attention kind: head h of H has the slope 2^(-8 (h + 1) / H)
SUTUVIK_SLOPE_EXPONENT = 8.0


def _sutuvik_layer(i: int, lc: dict) -> LayerSpec:
    m = lc["mixer"]
    kind = lc.get("type")
    if kind in ("attention", "attention_2"):
        kw = dict(mixer=MIXER_ATTENTION, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]),
                  vdim=int(m.get("vdim") or m["dim"]), scale=float(m["scale"]), sink=1, v_mix=int(bool(m.get("v_mix"))))
        if kind == "attention":
            qt = m.get("q_temp") or {}
            kw.update(qk_norm=3, dist_slope=SUTUVIK_SLOPE_EXPONENT, sink_learned=1, head_gate=1,
                      qtemp_coef=float(qt.get("coef") or 0.0), qtemp_every=int(qt.get("every") or 0))
        else:
            rot = m.get("rot") or {}
            sc = rot.get("scaling") or {}
            kw.update(qk_norm=1, head_temp=1, softcap=float(m.get("softcap") or 0.0), rot_pairs=1,
                      rot_dims=int(rot.get("dims") or 0), rot_base=float(rot.get("base") or 0.0))
            if sc:
                kw.update(rot_piecewise=1, rot_factor=float(sc["factor"]), rot_original=float(sc["original"]),
                          rot_fast=float(sc["high"]), rot_slow=float(sc["low"]))
    elif kind == "mamba2":
        kw = dict(mixer=MIXER_MAMBA2, heads=int(m["heads"]), vdim=int(m["vdim"]), dim=int(m["state"]),
                  state=int(m["state"]), ssm_groups=int(m.get("groups") or 1), norm_groups=int(m.get("norm_groups") or 1),
                  conv=int(m["conv"]))
    else:
        raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    mlp = lc.get("mlp")
    if mlp is None:
        pass
    elif mlp["kind"] == "moe":
        r = mlp["router"]
        g = r.get("groups") or {}
        kw.update(mlp=MLP_MOE, act=FFN_SWIGLU, ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]),
                  groups=int(g.get("count") or 0), keep_groups=int(g.get("keep") or 0), route_sigmoid=1,
                  route_correction=1, group_top2=1, route_norm=1)
    else:
        raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
    return LayerSpec(**kw)


def sutuvik_from_json(j: dict) -> ListedModelConfig:
    """config.json of the Sutuvik design: attention layers of two kinds and Mamba-2 layers in any
    order, pre-norm blocks whose norms work on equal parts of the row, a short causal convolution
    added to what every mixer reads, sigmoid-routed gated experts chosen within the best groups,
    a per-layer token input after the feed-forward, a normed embedding, logits through the
    embedding table times a constant."""
    nm = j["norm"]
    return ListedModelConfig(
        name="sutuvik", vocab_size=int(j["vocab"]), hidden=int(j["width"]),
        layers=tuple(_sutuvik_layer(i, lc) for i, lc in enumerate(j["layers"])),
        norm_eps=float(nm["eps"]), arch=ARCH_SUTUVIK, block_style=LBLOCK_SEQUENTIAL_PRENORM, tied_head=True,
        norm_groups=int(nm.get("groups") or 1), embed_norm=True,
        mixer_conv=int((j.get("canon") or {}).get("taps") or 0),
        side_dim=int((j.get("token_side") or {}).get("dim") or 0),
        logit_scale=float(j.get("logit_scale") or 0.0))


def safetensors_shapes(model_dir: str) -> dict:
    """Tensor name -> shape from the header of model.safetensors (8-byte little-endian length,
    then that many bytes of JSON)."""
    path = os.path.join(model_dir, "model.safetensors")
    if not os.path.exists(path):
        return {}
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        hdr = json.loads(f.read(n))
    return {k: tuple(v["shape"]) for k, v in hdr.items() if k != "__metadata__"}


# model registry: config.json "architecture" -> config builder
ARCHITECTURES = {"Dugopel": dugopel_from_json, "Zozonex": zozonex_from_json, "Lazovik": lazovik_from_json,
                 "Sutuvik": sutuvik_from_json}
# builders that also want the checkpoint's tensor shapes
_WANTS_SHAPES = {"Lazovik"}


def from_model_dir(model_dir: str):
    """The model class a directory's config.json names."""
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    arch = j.get("architecture")
    if arch not in ARCHITECTURES:
        raise ValueError(f"config.json names architecture {arch!r}; known: {sorted(ARCHITECTURES)}")
    if arch in _WANTS_SHAPES:
        return ARCHITECTURES[arch](j, safetensors_shapes(model_dir))
    return ARCHITECTURES[arch](j)
