"""Sutuvik (layers listed in config.json: two kinds of grouped-query attention with sinks — one
with weighted q / k norms, a query multiplier that grows with the position, a penalty linear in
the distance, a learned sink and a gate per head; one with rotated pairs, weightless norms, a
multiplier per head and capped scores —, values mixed with the first such layer's, Mamba-2 layers;
norms over equal parts of the row, a short convolution added to what every mixer reads, gated
experts routed by sigmoid scores within the best groups, a per-layer token input) against the plain
float64 restatement in tests/sutuvik_ref.py.  Every test makes its own small configuration and
random weights."""
import copy
import json
import os
import subprocess

import numpy as np
import pytest

from helpers import C, E, W, ROOT
import nvllm_pkg
import sutuvik_ref as ref
from st_writer import write_safetensors
from test_zozonex import Engine, prompt
from test_lazovik import check

gpu = pytest.mark.gpu
BLOCK = C.KV_BLOCK_SIZE
PRECS = [C.PREC_FP32, C.PREC_BF16]


# ------------------------------------------------------------------ configurations
def att(heads=4, kv_heads=2, dim=16, vdim=24, coef=0.4, every=7, scale=None, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5 if scale is None else scale),
         "v_mix": v_mix}
    if coef:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


STEPS = {"factor": 8.0, "original": 64, "high": 4.0, "low": 1.0}


def att2(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=10000.0, scaling=STEPS, scale=None, softcap=6.0, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5 if scale is None else scale),
         "v_mix": v_mix}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention_2", "mixer": m}


def mam(heads=4, vdim=12, state=8, groups=2, norm_groups=2, conv=4):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def moe(ff=32, experts=8, top=2, count=4, keep=2):
    r = {"experts": experts, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def layer(mix, mlp=None):
    return dict(copy.deepcopy(mix), mlp=mlp)


def model(layers, vocab=211, width=72, eps=1e-5, parts=3, taps=3, side=10, logit_scale=1.7):
    j = {"architecture": "Sutuvik", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": parts}, "layers": layers}
    if taps:
        j["canon"] = {"taps": taps}
    if side:
        j["token_side"] = {"dim": side}
    if logit_scale:
        j["logit_scale"] = logit_scale
    return j


def mixed_model():
    """All three mixers, with and without feed-forward, sizes that differ from layer to layer; the
    first value-mixing layer is of the rotated kind and not the model's first layer; a layer that
    mixes no values between two that do."""
    return model([layer(mam(), moe()),
                  layer(att2(v_mix=True), moe(ff=24, experts=6, top=1, count=3, keep=1)),
                  layer(att(v_mix=False, heads=6, kv_heads=3, dim=8, vdim=8, coef=0.9, every=3)),
                  layer(att(heads=2), moe(ff=40, experts=9, top=3, count=0)),
                  layer(mam(heads=2, vdim=24, state=16, groups=1, norm_groups=1, conv=2), moe(top=4, count=2, keep=2)),
                  layer(att2(heads=6, rot_dims=16, scaling=None, softcap=30.0), moe(experts=4, top=2, count=2, keep=1))])


def odd_model():
    """Sizes that are multiples of nothing convenient; whole-row norms; no convolution on the mixers'
    input, no token input, no logit multiplier; one-tap Mamba convolution; every entry rotated; no
    cap; no position multiplier; groups of two experts."""
    return model([layer(att2(heads=3, kv_heads=3, dim=20, vdim=12, rot_dims=20, base=77.0, scaling=None, softcap=0.0, v_mix=False),
                        moe(ff=20, experts=6, top=1, count=3, keep=2)),
                  layer(mam(heads=5, vdim=6, state=12, groups=5, norm_groups=3, conv=1), moe(ff=44, experts=7, top=7, count=0)),
                  layer(att(heads=5, kv_heads=1, dim=6, vdim=36, coef=0.0)),
                  layer(att2(heads=1, kv_heads=1, dim=36, vdim=4, rot_dims=2, v_mix=False))],
                 vocab=101, width=40, eps=3e-4, parts=1, taps=0, side=0, logit_scale=0.0)


def mma_model():
    """Head sizes that take the tensor-core attention kernels in bf16, grouped heads, unequal key and
    value sizes; Mamba-2 at sizes of a real model's heads."""
    return model([layer(att(heads=4, kv_heads=2, dim=64, vdim=64, every=16), moe(ff=64)),
                  layer(mam(heads=4, vdim=64, state=64, groups=1, norm_groups=4)),
                  layer(att2(heads=4, kv_heads=2, dim=128, vdim=64, rot_dims=64), moe(ff=96, experts=4, top=1, count=2, keep=1)),
                  layer(att(heads=2, kv_heads=2, dim=128, vdim=64, coef=0.2, every=100)),
                  layer(att2(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, scaling=None))],
                 width=128, parts=2, taps=4, side=16)


def tc5_model():
    """Keys and values of one size, 64, and scores neither capped nor biased by the distance in
    every attention layer: in bf16 the prefill steps of such a model run on the tcgen05 attention
    kernel with tiles of 128 queries (the sink joins there too)."""
    return model([layer(att2(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, softcap=0.0), moe(ff=64)),
                  layer(mam(heads=4, vdim=32, state=64, groups=1, norm_groups=4)),
                  layer(att2(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=64, scaling=None, softcap=0.0),
                        moe(ff=96, experts=4, top=1, count=2, keep=1)),
                  layer(att2(heads=2, kv_heads=2, dim=64, vdim=64, rot_dims=0, softcap=0.0))], width=128, parts=2, taps=4, side=16)


def random_weights(j, seed, bf16=False):
    cfg = C.sutuvik_from_json(j)
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in cfg.tensor_shapes().items():
        if name.endswith(".conv") or name.endswith(".canon1"):
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif name.endswith(".A_log"):
            a = rng.uniform(-3.0, 0.5, shape)     # with the step sizes below: decays per token from 0.2 to 0.999
        elif name.endswith(".dt_bias"):
            a = rng.uniform(-3.0, 0.0, shape)
        elif name.endswith(".D"):
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif name.endswith(".sink"):
            a = rng.standard_normal(shape)
        elif name.endswith(".temp"):
            a = rng.uniform(0.5, 2.0, shape)
        elif name.endswith(".vmix"):
            a = rng.uniform(0.2, 0.8, shape)
        elif name.endswith(".correction"):
            a = 0.3 * rng.standard_normal(shape)  # as large as the spread of the scores: the choice is not the ranking of the weights
        elif name.endswith(".conv.b"):
            a = 0.3 * rng.standard_normal(shape)
        elif len(shape) == 1:
            a = 1.0 + 0.2 * rng.standard_normal(shape)  # norm weights
        elif name in ("embed", "side.embed"):
            a = rng.standard_normal(shape)
        elif name.endswith(".g") or name.endswith(".router"):
            a = 2.0 * rng.standard_normal(shape) / np.sqrt(shape[1])
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        a = np.asarray(a, dtype=np.float32)
        w[name] = W.bf16_round(a) if bf16 else a
    return cfg, w


def setup(j, prec, seed=7, **kw):
    cfg, w = random_weights(j, seed, bf16=prec == C.PREC_BF16)
    return cfg, w, Engine(cfg, w, prec, **kw)


def no_close_calls(j, prec):
    """With random weights, some token in a few hundred has two choice scores closer than bf16
    rounding, and a run that then picks the other expert is not comparable from that token on.
    The bf16 runs of models with several layers therefore choose ALL experts of a layer (no
    groups; the scores still weight them); the choice is tested in fp32 and, in bf16, on single layers."""
    if prec == C.PREC_FP32:
        return j
    j = copy.deepcopy(j)
    for lc in j["layers"]:
        if lc.get("mlp"):
            lc["mlp"]["router"]["top"] = lc["mlp"]["router"]["experts"]
            lc["mlp"]["router"].pop("groups", None)
    return j


def routed(j):
    return any(lc.get("mlp") for lc in j["layers"])


# ------------------------------------------------------------------ CPU: configuration, the restatement itself
def test_config_reader_takes_every_size_and_constant_from_the_file():
    j = mixed_model()
    cfg = C.ARCHITECTURES[j["architecture"]](j)
    assert cfg.arch == C.ARCH_SUTUVIK and cfg.tied_head and cfg.needs_state_slots
    assert cfg.block_style == C.LBLOCK_SEQUENTIAL_PRENORM
    assert (cfg.norm_groups, cfg.mixer_conv, cfg.side_dim, cfg.embed_norm) == (3, 3, 10, True) and abs(cfg.logit_scale - 1.7) < 1e-12
    assert [l.mixer for l in cfg.layers] == [C.MIXER_MAMBA2, C.MIXER_ATTENTION, C.MIXER_ATTENTION, C.MIXER_ATTENTION,
                                             C.MIXER_MAMBA2, C.MIXER_ATTENTION]
    m0, a1, a2, a3, m4, a5 = cfg.layers
    assert (m0.heads, m0.vdim, m0.state, m0.ssm_groups, m0.norm_groups, m0.conv) == (4, 12, 8, 2, 2, 4)
    assert (m4.state, m4.ssm_groups, m4.norm_groups, m4.conv) == (16, 1, 1, 2)
    assert (a1.qk_norm, a1.rot_pairs, a1.rot_piecewise, a1.rot_dims, a1.head_temp, a1.sink, a1.sink_learned, a1.head_gate) == (1, 1, 1, 8, 1, 1, 0, 0)
    assert (a1.rot_factor, a1.rot_original, a1.rot_fast, a1.rot_slow, a1.softcap, a1.dist_slope) == (8.0, 64.0, 4.0, 1.0, 6.0, 0.0)
    assert (a2.qk_norm, a2.sink_learned, a2.head_gate, a2.v_mix, a2.qtemp_every, a2.dist_slope) == (3, 1, 1, 0, 3, 8.0) and abs(a2.qtemp_coef - 0.9) < 1e-12
    assert (a3.v_mix, a3.heads, a3.kv_heads) == (1, 2, 2) and (a5.rot_piecewise, a5.rot_dims, a5.softcap) == (0, 16, 30.0)
    assert (m0.experts, m0.top, m0.groups, m0.keep_groups, m0.route_sigmoid, m0.route_correction, m0.group_top2, m0.route_norm) == (8, 2, 4, 2, 1, 1, 1, 1)
    assert a2.mlp == C.MLP_NONE and (a3.experts, a3.top, a3.groups) == (9, 3, 0)
    sh = cfg.tensor_shapes()
    assert sh["embed"] == (211, 72) and "head" not in sh and sh["embed.norm"] == (72,) and sh["side.embed"] == (211, 60)
    assert sh["l0.mix.in"] == (2 * 48 + 2 * 16 + 4, 72) and sh["l0.mix.conv"] == (48 + 32, 4) and sh["l4.canon1"] == (72, 3)
    assert sh["l1.mix.temp"] == (4,) and sh["l1.mix.vmix"] == () and "l2.mix.vmix" not in sh and "l1.mix.sink" not in sh
    assert sh["l2.mix.q.norm"] == (8,) and sh["l2.mix.g"] == (6, 72) and "l2.norm2" not in sh and sh["l3.mlp.e8.down"] == (72, 40)
    assert sh["l5.side.gate"] == (10, 72) and sh["l5.side.proj"] == (72, 10) and sh["l3.mlp.correction"] == (9,)
    c, specs = cfg.to_c(C.PREC_FP32, num_state_slots=3)
    assert (c.norm_groups, c.embed_norm, c.mixer_conv, c.side_dim, c.num_state_slots) == (3, 1, 3, 10, 3)
    assert specs[2].qtemp_every == 3 and specs[0].state == 8 and specs[1].rot_pairs == 1
    # what the file does not mention does not exist
    o = C.sutuvik_from_json(odd_model())
    assert (o.norm_groups, o.mixer_conv, o.side_dim, o.logit_scale) == (1, 0, 0, 0.0)
    assert o.layers[0].softcap == 0.0 and o.layers[2].qtemp_coef == 0.0 and o.layers[0].rot_piecewise == 0
    assert "l0.canon1" not in o.tensor_shapes() and "side.embed" not in o.tensor_shapes()
    with pytest.raises(ValueError):
        C.sutuvik_from_json(model([dict(type="conv", mixer=att()["mixer"], mlp=None)]))
    with pytest.raises(ValueError):
        C.sutuvik_from_json(model([layer(att(), {"kind": "dense", "ff": 8})]))


def test_reference_mechanisms_against_hand_computed_values():
    """The restatement itself, on inputs small enough to check by hand."""
    x = np.array([[3.0, 4.0, 0.0, 2.0]])
    got = ref.rms_parts(x, np.array([1.0, 1.0, 1.0, 2.0]), 2, 0.0)
    assert np.allclose(got, [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5), 0.0, 2 * 2 / np.sqrt(2.0)]])
    u = np.array([[1.0], [2.0], [4.0]])
    assert ref.causal_conv(u, np.array([[10.0, 1.0]])).ravel().tolist() == [1.0, 12.0, 24.0]
    assert ref.causal_conv(u, np.array([[10.0, 1.0]]), np.array([0.5])).ravel().tolist() == [1.5, 12.5, 24.5]
    # a sink of score 0 beside one key of score 0 halves its weight; a hidden key weighs nothing
    p = ref.softmax_with_sink(np.array([[0.0, -np.inf]]), 0.0)
    assert np.allclose(p, [[0.5, 0.0]])
    # one head, state 1 x 1: decay exp(-exp(0) * 1) = 1 / e per token, input dt * B * x
    y = ref.state_space_scan(np.ones((2, 1, 1)), np.ones((2, 1, 1)), np.ones((2, 1, 1)), np.ones((2, 1)), np.zeros(1), np.array([2.0]), 1)
    assert np.allclose(y.ravel(), [1.0 + 2.0, np.exp(-1.0) + 1.0 + 2.0])
    f = ref.rotation_frequencies({"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 8, "high": 4.0, "low": 1.0}})
    # wavelengths 2 pi (> 2, < 8: blended with s = (8 / 2 pi - 1) / 3) and 20 pi (> 8: divided)
    s = (8 / (2 * np.pi) - 1.0) / 3.0
    assert np.allclose(f, [(1 - s) * 0.5 + s, 0.1 / 2.0])
    r = ref.rotate_pairs(np.array([[[1.0, 0.0, 5.0]]]), np.array([np.pi / 2]), np.array([1.0]))
    assert np.allclose(r, [[[0.0, 1.0, 5.0]]])
    # choice: group 1 holds the best single expert, group 0 the best pair; the correction decides, the weights ignore it
    router = {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}
    sc = np.array([0.5, 0.6, 0.9, 0.1])
    assert ref.choose_experts(sc, np.zeros(4), router) == [1, 0]
    assert ref.choose_experts(sc, np.array([0.0, 0.0, 0.0, 0.3]), router) == [2, 3]
    # negative scores: group 1 (-1.0 against -1.1) is kept; were hidden experts zeros, expert 0 would win
    assert ref.choose_experts(-sc, np.zeros(4), dict(router, top=1)) == [3]
    assert ref.choose_experts(sc, np.zeros(4), {"experts": 4, "top": 2}) == [2, 1]


# ------------------------------------------------------------------ GPU: each mechanism alone
BARE = dict(parts=1, taps=0, side=0, logit_scale=0.0)
CASES = {
    "attention_biased": lambda: model([layer(att(v_mix=False))], **BARE),
    "attention_biased_plain": lambda: model([layer(att(v_mix=False, coef=0.0, heads=3, kv_heads=3))], **BARE),
    "attention_rotary": lambda: model([layer(att2(v_mix=False))], **BARE),
    "attention_rotary_plain": lambda: model([layer(att2(v_mix=False, rot_dims=0, softcap=0.0))], **BARE),
    "attention_rotary_all_entries": lambda: model([layer(att2(v_mix=False, rot_dims=16, scaling=None, base=50.0))], **BARE),
    "attention_biased_heads_of_128": lambda: model([layer(att(heads=4, kv_heads=1, dim=128, vdim=128, v_mix=False, every=20))], **dict(BARE, width=128)),
    "attention_rotary_heads_of_128": lambda: model([layer(att2(heads=2, kv_heads=2, dim=128, vdim=128, v_mix=False, rot_dims=96, softcap=0.0))], **dict(BARE, width=128)),
    "attention_rotary_heads_of_64": lambda: model([layer(att2(heads=6, kv_heads=2, dim=64, vdim=64, v_mix=False, rot_dims=64, softcap=0.0))], **dict(BARE, width=128)),
    "value_mixing": lambda: model([layer(att()), layer(att2()), layer(att())], **BARE),
    "mamba2": lambda: model([layer(mam())], **BARE),
    "mamba2_one_group_wide_state": lambda: model([layer(mam(heads=2, vdim=40, state=200, groups=1, norm_groups=1, conv=3))], **BARE),
    "mamba2_every_head_its_group": lambda: model([layer(mam(heads=3, vdim=8, state=4, groups=3, norm_groups=6, conv=8))], **BARE),
    "norm_in_parts": lambda: model([layer(att(v_mix=False))], **dict(BARE, parts=9)),
    "mixer_input_convolution": lambda: model([layer(att(v_mix=False)), layer(mam())], **dict(BARE, taps=5)),
    "token_input": lambda: model([layer(att(v_mix=False)), layer(mam())], **dict(BARE, side=5)),
    "logit_multiplier": lambda: model([layer(mam())], **dict(BARE, logit_scale=0.25)),
    "experts_in_groups": lambda: model([layer(att(v_mix=False), moe(ff=20, experts=12, top=3, count=4, keep=2))], **BARE),
    "experts_one_group_kept": lambda: model([layer(mam(), moe(ff=12, experts=10, top=2, count=5, keep=1))], **BARE),
    "experts_no_groups": lambda: model([layer(att2(v_mix=False), moe(ff=200, experts=5, top=5, count=0))], **BARE),
    "everything": lambda: model([layer(att(), moe()), layer(mam(), moe()), layer(att2(), moe())]),
}


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("case", sorted(CASES))
def test_each_mechanism_alone(case, prec):
    j = CASES[case]()
    if case == "everything":
        j = no_close_calls(j, prec)
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 90, 1)
        got, _ = eng.step([("a", toks, list(range(90)))])
        check(got, ref.forward(j, w, toks), prec, case, routed(j))
    finally:
        eng.close()


@gpu
def test_residual_stream_after_every_layer():
    """One layer more, one more entry of the reference's stream to meet: models of 1 .. n layers
    share their first layers' weights, the last layer's output is read through norm and table."""
    full = mixed_model()
    cfgf, wf = random_weights(full, 9)
    toks = prompt(full, 50, 2)
    for n in range(1, len(full["layers"]) + 1):
        j = dict(full, layers=full["layers"][:n])
        cfg = C.sutuvik_from_json(j)
        w = {k: wf[k] if k != "side.embed" else wf[k][:, :n * 10] for k in cfg.tensor_shapes()}
        eng = Engine(cfg, w, C.PREC_FP32)
        try:
            got, _ = eng.step([("a", toks, list(range(50)))])
            check(got, ref.forward(j, w, toks), C.PREC_FP32, f"{n} layers")
        finally:
            eng.close()


MODELS = {"mixed": mixed_model, "odd": odd_model, "mma": mma_model, "tc5": tc5_model}


# ------------------------------------------------------------------ GPU: schedules
@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("which", sorted(MODELS))
def test_prefill_equals_token_by_token_decoding(which, prec):
    j = no_close_calls(MODELS[which](), prec)
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 70, 2)
        want = ref.forward(j, w, toks)
        got, _ = eng.step([("whole", toks, list(range(70)))])
        check(got, want, prec, "whole prompt", True)
        rows = [eng.step([("dec", toks[:9], [8])])[0][0]]
        for t in range(9, 70):
            rows.append(eng.step([("dec", [toks[t]], [0])], decode=True)[0][0])
        check(np.stack(rows), want[8:], prec, "decoded", True)
        if prec == C.PREC_FP32:  # the same arithmetic either way: far closer to each other than to float64
            assert np.abs(np.stack(rows) - got[8:]).max() <= 2e-5 * np.abs(want).max()
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("which", ["mixed", "mma", "tc5"])
def test_portions_of_several_sizes_down_to_two_tokens(which, prec):
    j = no_close_calls(MODELS[which](), prec)
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 331, 3)
        want = ref.forward(j, w, toks)
        got, pos = [], 0
        # portions shorter than either convolution, one token, one that crosses the page border at 256
        for n in [2, 3, 2, 16, 17, 40, 1, 5, 100, 2, 71, 2, 70]:
            out, _ = eng.step([("p", toks[pos:pos + n], list(range(n)))])
            got.append(out)
            pos += n
        assert pos == 331
        check(np.concatenate(got), want, prec, "portions", True)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("which,prec", [("mixed", C.PREC_FP32), ("mma", C.PREC_BF16), ("tc5", C.PREC_BF16)])
def test_batches_of_unequal_requests_equal_each_alone(which, prec):
    j = no_close_calls(MODELS[which](), prec)
    cfg, w, eng = setup(j, prec, num_blocks=10)
    try:
        A, B, Cc, Dd = (prompt(j, n, s) for n, s in ((150, 4), (41, 5), (7, 6), (290, 7)))
        wa, wb, wc, wd = (ref.forward(j, w, t) for t in (A, B, Cc, Dd))
        g1, _ = eng.step([("a", A[:100], [0, 99]), ("b", B, [40]), ("c", Cc[:2], [1])])
        g2, _ = eng.step([("c", Cc[2:], [4]), ("a", A[100:], [49]), ("b", [3], [0]), ("d", Dd[:260], [255, 256, 259])])
        wb2 = ref.forward(j, w, B + [3])
        g3, _ = eng.step([("d", [Dd[260]], [0]), ("a", [9], [0]), ("c", [11], [0])], decode=True)
        got = np.concatenate([g1, g2, g3])
        want = np.stack([wa[0], wa[99], wb[40], wc[1], wc[6], wa[149], wb2[41], wd[255], wd[256], wd[259], wd[260],
                         ref.forward(j, w, A + [9])[150], ref.forward(j, w, Cc + [11])[7]])
        check(got, want, prec, "three steps", True)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_pages_and_slots_are_freed_and_used_again(prec):
    j = no_close_calls(mixed_model(), prec)
    cfg, w, eng = setup(j, prec, num_blocks=3, slots=2)
    try:
        got, want = [], []
        for r in range(5):  # 5 pairs of requests through 2 slots and 3 pages; each leaves state, tails, keys and values behind
            a, b = prompt(j, 200 + 20 * r, 10 + r), prompt(j, 30 + r, 20 + r)
            ga, _ = eng.step([("a", a[:120], [119]), ("b", b[:10], [9])])
            gb, _ = eng.step([("a", a[120:], [len(a) - 121]), ("b", b[10:], [len(b) - 11])])
            wa, wb = ref.forward(j, w, a), ref.forward(j, w, b)
            got += [ga, gb]
            want += [wa[119], wb[9], wa[-1], wb[-1]]
            if r % 2:
                eng.end("a"), eng.end("b")
            else:
                eng.end("b"), eng.end("a")
        check(np.concatenate(got), np.stack(want), prec, "five rounds", True)
        assert len(eng.bm.free_block_ids) == 3 and len(eng.bm.free_state_slots) == 2
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("which,prec", [("odd", C.PREC_FP32), ("mixed", C.PREC_FP32), ("mixed", C.PREC_BF16), ("mma", C.PREC_BF16),
                                        ("tc5", C.PREC_BF16)])
def test_first_tokens_of_a_sequence(which, prec):
    """Positions 0, 1, 2: shorter than the convolutions and any tile; a one-token prompt (its only
    key shares the softmax with the sink); the convolutions read zeros before the start and the
    state begins at zero, whatever the slot held."""
    j = no_close_calls(MODELS[which](), prec)
    cfg, w, eng = setup(j, prec)
    try:
        eng.step([("dirt", prompt(j, 40, 29), [])])  # leaves state, tails and keys in slot and page
        eng.end("dirt")
        for n in (1, 2, 3):
            toks = prompt(j, n, 30 + n)
            got, _ = eng.step([("s", toks, list(range(n)))])
            nxt, _ = eng.step([("s", [4], [0])], decode=True)
            want = ref.forward(j, w, toks + [4])
            check(np.concatenate([got, nxt]), want, prec, f"{n} tokens + 1")
            eng.end("s")
    finally:
        eng.close()


@gpu
def test_long_decoding_stays_on_the_reference():
    j = mixed_model()
    cfg, w, eng = setup(j, C.PREC_FP32)
    try:
        toks = prompt(j, 560, 40)
        want = ref.forward(j, w, toks)
        eng.step([("l", toks[:20], [])])
        rows = [eng.step([("l", [toks[t]], [0])], decode=True)[0][0] for t in range(20, 560)]
        check(np.stack(rows), want[20:], C.PREC_FP32, "540 decoded tokens")
    finally:
        eng.close()


# ------------------------------------------------------------------ GPU: faults that random weights would hide
BIG = 5


def make_standout(w, rows_of, gain):
    """Every sublayer norms what it reads, so a token cannot stand out by the size of its embedding.
    Instead: entry 0 of every embedding is zero except token BIG's, which is nothing else, and
    column 0 of the given projection rows is multiplied by `gain` — what token BIG (and only it)
    sends through those rows is that much larger than any other token's."""
    w["embed"][:, 0] = 0.0
    w["embed"][BIG] = 0.0
    w["embed"][BIG, 0] = 8.0
    for name, rows in rows_of:
        w[name][rows, 0] *= gain
    return w


def without(toks, t=BIG, other=6):
    return [other if x == t else x for x in toks]


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("kind", ["biased", "rotary"])
def test_a_far_key_among_hundreds(kind, prec):
    """Attention layers only.  One token's value is hundreds of times the others'; it sits at
    position 3 and is read from hundreds of positions later, over page borders, in a prompt's
    portions and in decoding.  (Under the distance penalty only the heads with the gentlest slopes
    still see it, from 300 positions away.)"""
    d = 64 if prec == C.PREC_BF16 else 16
    if kind == "biased":
        mk, n = (lambda: layer(att(heads=8, kv_heads=2, dim=d, vdim=d, v_mix=False, every=50))), 330
    else:
        # (bf16: uncapped scores, the tcgen05 prefill kernel)
        mk, n = (lambda: layer(att2(heads=2, kv_heads=1, dim=d, vdim=d, v_mix=False, rot_dims=8, softcap=0.0 if d == 64 else 6.0))), 880
    j = model([mk(), mk()], width=64, parts=2, side=0)
    cfg, w = random_weights(j, 14, bf16=prec == C.PREC_BF16)
    make_standout(w, [("l0.mix.v", slice(None))], 400.0)
    eng = Engine(cfg, w, prec)
    try:
        base = without(prompt(j, n, 15))
        far = list(base)
        far[3] = BIG
        plain, want = ref.forward(j, w, base), ref.forward(j, w, far)
        assert np.abs(want[n - 20:] - plain[n - 20:]).max() > 0.05 * np.abs(plain).max()  # the test's own premise
        got, pos = [], 0
        cuts = [250, 12, n - 30 - 262]
        for c in cuts:
            out, _ = eng.step([("f", far[pos:pos + c], [0, c - 1])])
            got.append(out)
            pos += c
        rows = [eng.step([("f", [far[t]], [0])], decode=True)[0][0] for t in range(pos, n)]
        probes = [0, 249, 250, 261, 262, pos - 1] + list(range(pos, n))
        check(np.concatenate(got + [np.stack(rows)]), want[probes], prec, kind)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_a_far_token_reaches_through_the_recurrent_state(prec):
    """Mamba-2 layers only, decays near one: nothing but the carried state links position 600 to
    position 2.  The prompt goes in portions and then decodes, over two page borders."""
    j = model([layer(mam(heads=2, vdim=16, state=32, groups=1, norm_groups=1)), layer(mam(heads=4, vdim=8, state=16, groups=2))],
              width=64, parts=2, side=0)
    cfg, w = random_weights(j, 12, bf16=prec == C.PREC_BF16)
    for name in w:
        if name.endswith(".A_log"):
            w[name][:] = -7.0
    make_standout(w, [("l0.mix.in", slice(32, 64))], 300.0)  # the rows of x: the token's input to the state
    eng = Engine(cfg, w, prec)
    try:
        toks = without(prompt(j, 640, 13), other=8)
        with_far = list(toks)
        with_far[2] = BIG
        want, plain = ref.forward(j, w, with_far), ref.forward(j, w, toks)
        assert np.abs(want[600:] - plain[600:]).max() > 0.1 * np.abs(want[600:]).max()  # the test's own premise
        got, pos = [], 0
        for n in (250, 12, 200, 138):
            out, _ = eng.step([("f", with_far[pos:pos + n], [n - 1])])
            got.append(out[0])
            pos += n
        for t in range(600, 640):
            got.append(eng.step([("f", [with_far[t]], [0])], decode=True)[0][0])
        check(np.stack(got), want[[249, 261, 461, 599] + list(range(600, 640))], prec, "far token")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("kind", ["learned", "zero"])
def test_a_sink_that_outweighs_every_key(kind, prec):
    """The sink takes most of the softmax's mass: a learned sink of 4 beside scores near zero, or the
    sink of score zero beside scores that a small scale keeps far below it for the first tokens.
    Left out, counted per key, scaled or biased, the read-out would be several times too large
    (the logits, which also hold the token's own embedding, move by a tenth of their range)."""
    d = 64 if prec == C.PREC_BF16 else 16  # bf16: the tensor-core kernels' sizes
    if kind == "learned":
        j = model([layer(att(heads=4, kv_heads=2, dim=d, vdim=d, v_mix=False, scale=0.02))], **BARE)
    else:
        j = model([layer(att2(heads=4, kv_heads=2, dim=d, vdim=d, v_mix=False, scale=0.02, softcap=0.0 if d == 64 else 6.0))], **BARE)
    cfg, w = random_weights(j, 16, bf16=prec == C.PREC_BF16)
    if kind == "learned":
        w["l0.mix.sink"][:] = np.array([4.0, 3.0, 5.0, -2.0], dtype=np.float32)
    toks = prompt(j, 40, 17)
    want = ref.forward(j, w, toks)
    # the premise: without its sink the first layer's read-out differs grossly
    w0 = dict(w)
    if kind == "learned":
        w0["l0.mix.sink"] = np.full(4, -30.0, dtype=np.float32)
        assert np.abs(ref.forward(j, w0, toks) - want).max() > 0.05 * np.abs(want).max()
    eng = Engine(cfg, w, prec)
    try:
        got, _ = eng.step([("p", toks[:30], list(range(30)))])
        rows = [eng.step([("p", [toks[t]], [0])], decode=True)[0][0] for t in range(30, 40)]
        check(np.concatenate([got, np.stack(rows)]), want, prec, kind)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("every", [1, 64, 128])
def test_the_query_multiplier_steps_at_the_right_positions(every, prec):
    """q grows by the factor 1 + coef ln(floor((p + 1) / every) + 1): it first changes at position
    every - 1, then at 2 every - 1 (for every = 128: the last position of the first page).  With a
    coefficient of 3 and sharp scores a step taken one position early or late changes that row's
    logits grossly.  Probed inside a prompt and with the same positions decoded."""
    d = 64 if prec == C.PREC_BF16 else 16
    j = model([layer(att(heads=2, kv_heads=1, dim=d, vdim=d, coef=3.0, every=every, v_mix=False, scale=2.0 * d ** -0.5))],
              width=64, parts=2, side=0)
    cfg, w = random_weights(j, 18, bf16=prec == C.PREC_BF16)
    w["l0.mix.o"] *= 16.0  # the attention's read-out outweighs the token's own embedding in the logits
    n = 2 * every + 3 if every > 1 else 12
    toks = prompt(j, n, 19)
    want = ref.forward(j, w, toks)
    if every > 1:  # the premise: the step matters
        early = copy.deepcopy(j)
        early["layers"][0]["mixer"]["q_temp"]["every"] = every - 1
        assert np.abs(ref.forward(early, w, toks)[every - 2] - want[every - 2]).max() > 0.1 * np.abs(want).max()
    eng = Engine(cfg, w, prec)
    try:
        probes = sorted({0, 1, max(every - 2, 0), every - 1, every, 2 * every - 2, 2 * every - 1, 2 * every, n - 1})
        got, _ = eng.step([("p", toks, probes)])
        check(got, want[probes], prec, "prompt")
        eng.end("p")
        start = max(every - 3, 1)
        eng.step([("d", toks[:start], [])])
        rows = [eng.step([("d", [toks[t]], [0])], decode=True)[0][0] for t in range(start, n)]
        check(np.stack(rows), want[start:], prec, "decoded")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_the_correction_chooses_and_the_plain_scores_weigh(prec):
    """One layer, corrections as large as the scores themselves and of both signs, one group kept
    of four: an implementation that weighs with the corrected scores, ranks groups by their best
    expert alone, or treats hidden experts as zeros gives other logits."""
    j = model([layer(mam(), moe(ff=24, experts=12, top=2, count=4, keep=1))], **BARE)
    cfg, w = random_weights(j, 20, bf16=prec == C.PREC_BF16)
    w["l0.mlp.correction"][:] = W.bf16_round(np.random.default_rng(3).uniform(-1.5, 0.5, 12).astype(np.float32))
    toks = prompt(j, 120, 21)
    want = ref.forward(j, w, toks)
    eng = Engine(cfg, w, prec)
    try:
        got, _ = eng.step([("p", toks, list(range(120)))])
        check(got, want, prec, "routing", True)
    finally:
        eng.close()


@gpu
def test_decoding_with_the_keys_of_a_long_context_cut_into_ranges():
    """bf16, tensor-core head sizes, three sequences of 900, 300 and 5 tokens decoding together: a
    decode step cuts the keys of each (sequence, key / value head) into ranges that separate CTAs
    read, some of them empty for the short sequences; the sink must join the merged state once."""
    j = model([layer(att(heads=4, kv_heads=2, dim=64, vdim=64, every=100)), layer(att2(heads=8, kv_heads=2, dim=128, vdim=64, rot_dims=64)),
               layer(att(heads=2, kv_heads=2, dim=128, vdim=64, coef=0.0))], width=128, parts=2, side=8)
    cfg, w, eng = setup(j, C.PREC_BF16, seed=31, num_blocks=8)
    try:
        lens = {"a": 900, "b": 300, "c": 5}
        toks = {k: prompt(j, n + 12, 32 + i) for i, (k, n) in enumerate(lens.items())}
        want = {k: ref.forward(j, w, t) for k, t in toks.items()}
        eng.step([(k, toks[k][:n], []) for k, n in lens.items()])
        rows = {k: [] for k in lens}
        for t in range(12):
            out, _ = eng.step([(k, [toks[k][n + t]], [0]) for k, n in lens.items()], decode=True)
            for i, k in enumerate(lens):
                rows[k].append(out[i])
        for k, n in lens.items():
            check(np.stack(rows[k]), want[k][n:], C.PREC_BF16, f"sequence {k}")
    finally:
        eng.close()


# ------------------------------------------------------------------ GPU: models drawn at random
def draw_model(rng):
    """Sizes, head counts, layer order, constants and which options exist at all are drawn."""
    layers = []
    kv_mix, vdim_mix = int(rng.integers(1, 4)), int(rng.choice([8, 16, 24, 64]))  # layers that mix values share these
    for _ in range(int(rng.integers(2, 7))):
        kind = rng.choice(["attention", "attention_2", "mamba2"])
        if kind == "mamba2":
            g = int(rng.choice([1, 2, 3]))
            heads, vdim = g * int(rng.integers(1, 4)), int(rng.choice([4, 8, 16, 32, 64]))
            parts = [p for p in (1, 2, 4, heads) if (heads * vdim) % p == 0]
            mix = mam(heads=heads, vdim=vdim, state=int(rng.choice([4, 8, 16, 32, 64, 128])), groups=g,
                      norm_groups=int(rng.choice(parts)), conv=int(rng.integers(1, 6)))
        else:
            v_mix = bool(rng.random() < 0.6)
            kv = kv_mix if v_mix else int(rng.integers(1, 5))
            heads = kv * int(rng.choice([1, 2, 3, 4]))
            dim = int(rng.choice([8, 16, 32, 48, 64, 128]))
            vdim = vdim_mix if v_mix else int(rng.choice([8, 16, 32, 64, 128]))
            scale = float(dim ** -0.5 * rng.uniform(0.5, 2))
            if kind == "attention":
                mix = att(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, coef=0.0 if rng.random() < 0.3 else float(rng.uniform(0.1, 1.0)),
                          every=int(rng.integers(1, 100)), scale=scale, v_mix=v_mix)
            else:
                sc = None if rng.random() < 0.4 else {"factor": float(rng.uniform(1.5, 8)), "original": int(rng.integers(16, 4096)),
                                                      "high": float(rng.uniform(4, 64)), "low": float(rng.uniform(0.5, 2))}
                mix = att2(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, rot_dims=int(rng.integers(0, dim // 2 + 1)) * 2,
                           base=float(rng.choice([100.0, 10000.0, 500000.0])), scaling=sc, scale=scale,
                           softcap=float(rng.choice([0.0, 5.0, 20.0, 50.0])), v_mix=v_mix)
        mlp = None
        if rng.random() < 0.8:
            count = int(rng.choice([0, 1, 2, 3, 4]))
            per = int(rng.integers(2, 6))
            e = (count or 1) * per
            keep = int(rng.integers(1, count + 1)) if count else 0
            top = int(rng.integers(1, min(4, (keep or 1) * per) + 1))
            mlp = moe(ff=int(rng.integers(8, 100)), experts=e, top=top, count=count, keep=keep)
        layers.append(layer(mix, mlp))
    width = int(rng.choice([64, 96, 128, 192, 256]))
    return model(layers, vocab=int(rng.integers(50, 500)), width=width, eps=float(rng.choice([1e-5, 1e-6, 1e-4])),
                 parts=int(rng.choice([1, 2, 4, 8])), taps=int(rng.choice([0, 2, 3, 4, 6])),
                 side=int(rng.choice([0, 3, 8, 16, 20])), logit_scale=float(rng.choice([0.0, 0.5, 3.0])))


@gpu
@pytest.mark.parametrize("seed", range(8))
def test_models_drawn_at_random(seed):
    """Whole prompt, then the same tokens in drawn portions with the last ones decoded, beside a
    second request that comes and goes; fp32, every row."""
    rng = np.random.default_rng(5000 + seed)
    j = draw_model(rng)
    cfg, w, eng = setup(j, C.PREC_FP32, seed=50 + seed)
    try:
        n = int(rng.integers(30, 330))
        toks, other = prompt(j, n, 60 + seed), prompt(j, int(rng.integers(3, 120)), 70 + seed)
        want, want_o = ref.forward(j, w, toks), ref.forward(j, w, other)
        got, _ = eng.step([("w", toks, list(range(n)))])
        check(got, want, C.PREC_FP32, "whole prompt")
        eng.end("w")
        rows, pos, po, ndec = [], 0, 0, int(rng.integers(1, 9))
        while pos < n - ndec:
            c = int(min(n - ndec - pos, rng.choice([2, 2, 3, 5, 17, 64, 100, 130])))
            entries = [("p", toks[pos:pos + c], list(range(c)))]
            if po < len(other):
                co = int(min(len(other) - po, rng.choice([1, 2, 9, 40])))
                entries.append(("o", other[po:po + co], [co - 1]))
            out, _ = eng.step(entries)
            rows.append(out[:c])
            if len(entries) > 1:
                check(out[c:], want_o[po + co - 1:po + co], C.PREC_FP32, "second request")
                po += co
                if po >= len(other):
                    eng.end("o")
            pos += c
        for t in range(pos, n):
            rows.append(eng.step([("p", [toks[t]], [0])], decode=True)[0])
        check(np.concatenate(rows), want, C.PREC_FP32, "portions and decoding")
    finally:
        eng.close()


# ------------------------------------------------------------------ GPU: entry points
@gpu
def test_greedy_generation_through_the_engine_and_its_scheduler():
    """LLMEngine.generate: the scheduler admits the prompts, the block manager hands out pages
    and state slots, Run() samples greedily; three requests of unequal length at once."""
    R = nvllm_pkg.sub("runner")
    j = mixed_model()
    cfg, w = random_weights(j, 21)
    run = R.CudaModelRunner(cfg, w.items(), precision=C.PREC_FP32, num_kv_blocks=12, sampling=None, num_state_slots=8)
    eng = E.LLMEngine(E.EngineConfig(max_num_seqs=8, num_kvcache_blocks=12, max_model_len=4096), run)
    try:
        prompts = [prompt(j, n, 50 + n) for n in (5, 61, 250)]
        outs = eng.generate(prompts, E.SamplingParams(temperature=1.0, max_tokens=12, ignore_eos=True), temperature=0.0)
        for p, o in zip(prompts, outs):
            assert o == ref.greedy(j, w, p, 12)
        assert len(eng.scheduler.block_manager.free_state_slots) == 8
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_command_line_on_a_model_directory(tmp_path, dtype):
    """bin/trace_run: config.json + model.safetensors (bf16, the mixing weights as scalars) in,
    logits of the wanted places out."""
    j = no_close_calls(mixed_model(), C.PREC_FP32 if dtype == "float32" else C.PREC_BF16)
    cfg, w = random_weights(j, 22, bf16=True)
    mdir, out = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(j))
    write_safetensors(str(mdir / "model.safetensors"), w, dtype="BF16")
    a, b = prompt(j, 80, 60), prompt(j, 9, 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b, "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[50:], "want": [29]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [7], "want": [0]}, {"id": "c", "tokens": b[:4], "want": [3]}], "end": ["a", "c"]}]
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb, wa2 = ref.forward(j, w, a), ref.forward(j, w, b), ref.forward(j, w, a + [7])
    prec = C.PREC_FP32 if dtype == "float32" else C.PREC_BF16
    V = j["vocab"]
    got = np.concatenate([np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, V) for s in (0, 1, 2)])
    check(got, np.stack([wa[49], wb[0], wb[8], wa[79], wa2[80], wb[3]]), prec, "three steps", True)


@gpu
def test_sizes_the_kernels_do_not_cover_are_refused_at_create():
    L = nvllm_pkg.sub("lib")
    R = nvllm_pkg.sub("runner")
    for bad in ([layer(mam(heads=1, vdim=8, state=300, groups=1, norm_groups=1))],
                [layer(att(vdim=24)), layer(att(vdim=16))]):  # values of unequal sizes cannot be mixed
        cfg, w = random_weights(model(bad), 1)
        with pytest.raises(L.NvllmError):
            R.CudaModelRunner(cfg, w.items(), precision=C.PREC_FP32, num_kv_blocks=2, sampling=None, num_state_slots=1)
