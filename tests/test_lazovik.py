"""Lazovik (layers listed in config.json: gated linear attention, and a convolved / rotated /
score-capped / chunk-masked / gated attention beside time mixing with a token shift; pre-norm
blocks; sigmoid-routed squared-ReLU experts with an always-on expert; a run of layers that
repeats with state of its own per pass) against the plain float64 restatement in
tests/lazovik_ref.py.  Every test makes its own small configuration and random weights."""
import copy
import json
import os
import subprocess

import numpy as np
import pytest

from helpers import C, E, W, ROOT
import nvllm_pkg
import lazovik_ref as ref
from st_writer import write_safetensors
from test_zozonex import Engine, prompt

gpu = pytest.mark.gpu
BLOCK = C.KV_BLOCK_SIZE
PRECS = [C.PREC_FP32, C.PREC_BF16]


# ------------------------------------------------------------------ configurations
def gla(heads=3, dim=16, vdim=24, tau=8.0, rank=8):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "_rank": rank}}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def par(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, chunk=40, rot_dims=8, base=10000.0, scaling=YARN, scale=None,
        softcap=6.0, heads2=2, dim2=16, rank=8, ls=1.1, rs=0.7):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": chunk},
            "rot": {"base": base, "dims": rot_dims, "scaling": scaling}, "scale": float(dim ** -0.5 if scale is None else scale),
            "softcap": softcap}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": heads2, "dim": dim2, "_rank": rank},
                                          "left_scale": ls, "right_scale": rs}}


def moe(ff=32, experts=6, top=2, shared=48):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mix, mlp=None):
    return dict(copy.deepcopy(mix), mlp=mlp)


def model(layers, vocab=211, width=64, eps=1e-5, loop=None):
    j = {"architecture": "Lazovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        j["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return j


def mixed_model():
    """Both mixers, with and without feed-forward, sizes that differ from layer to layer, a
    repeated run in the middle (a layer before it, one after), three passes."""
    return model([layer(gla(), moe()),
                  layer(par(), moe(ff=24, experts=5, top=1, shared=0)),
                  layer(gla(heads=2, dim=24, vdim=8, tau=3.0, rank=4)),
                  layer(par(heads=6, kv_heads=1, dim=8, vdim=16, conv=2, chunk=23, rot_dims=4, scaling=None, softcap=30.0,
                            heads2=3, dim2=8, rank=5, ls=0.6, rs=1.3), moe(ff=40, experts=9, top=3, shared=16)),
                  layer(gla(heads=1, dim=32, vdim=32, tau=1.0, rank=16), moe(top=1))], loop=(1, 4, 3))


def odd_model():
    """Sizes that are multiples of nothing convenient, one-tap convolution, a chunk of one and a
    chunk longer than any prompt, every entry of a head rotated, no repeated run."""
    return model([layer(par(heads=3, kv_heads=3, dim=20, vdim=12, conv=1, chunk=1, rot_dims=20, heads2=1, dim2=36, rank=3),
                        moe(ff=20, experts=3, top=3, shared=28)),
                  layer(gla(heads=5, dim=12, vdim=10, tau=2.5, rank=7), moe(ff=44, experts=7, top=2, shared=0)),
                  layer(par(heads=5, kv_heads=1, dim=6, vdim=36, conv=4, chunk=5000, rot_dims=2, base=77.0, scaling=None,
                            heads2=5, dim2=4, rank=2))], vocab=101, width=40, eps=3e-4)


def mma_model():
    """Head sizes that take the tensor-core attention kernels in bf16, grouped heads, chunks that
    are no multiple of the key tile; recurrences at their largest compiled sizes."""
    return model([layer(par(heads=4, kv_heads=2, dim=64, vdim=64, chunk=100, rot_dims=32, heads2=2, dim2=64, rank=16), moe(ff=64)),
                  layer(gla(heads=2, dim=64, vdim=96, rank=16)),
                  layer(par(heads=4, kv_heads=1, dim=128, vdim=128, chunk=37, rot_dims=64, scaling=None, heads2=1, dim2=128),
                        moe(ff=96, experts=4, top=1, shared=64)),
                  layer(par(heads=2, kv_heads=2, dim=64, vdim=128, conv=2, chunk=64, rot_dims=64, heads2=1, dim2=200))],
                 width=128, loop=(0, 2, 2))


def shapes_of(j):
    """What a checkpoint's header would say about the sizes config.json does not hold."""
    W_ = j["width"]
    s = {}
    for i, lc in enumerate(j["layers"]):
        if lc["type"] == "gla":
            s[f"l{i}.mix.a1"] = (lc["mixer"]["_rank"], W_)
        else:
            s[f"l{i}.mix.right.w1"] = (lc["mixer"]["right"]["_rank"], W_)
    return s


def random_weights(j, seed, bf16=False):
    cfg = C.lazovik_from_json(j, shapes_of(j))
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in cfg.tensor_shapes().items():
        if name.endswith(".conv"):
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif name.endswith("a2.b"):
            a = rng.uniform(0.0, 4.0, shape)      # decays sigmoid(z)^(1 / tau) mostly near one
        elif name.endswith(".w0"):
            a = rng.uniform(-5.0, -0.5, shape)    # decays exp(-exp(z)) from 0.55 up
        elif name.endswith(".a2") or name.endswith(".w2"):
            a = 0.5 * rng.standard_normal(shape) / np.sqrt(shape[1])
        elif ".mu." in name:
            a = rng.uniform(0.0, 1.0, shape)
        elif name.endswith(".u") or name == "loop.step":
            a = 0.5 * rng.standard_normal(shape)
        elif name.endswith(".b"):
            a = 0.3 * rng.standard_normal(shape)
        elif len(shape) == 1:
            a = 1.0 + 0.2 * rng.standard_normal(shape)  # norm weights
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif name.endswith(".down"):
            # squared-ReLU experts square the relative error they are given; kept small beside the stream,
            # or a model of a dozen layer executions multiplies bf16 rounding by hundreds
            a = 0.3 * rng.standard_normal(shape) / np.sqrt(shape[1])
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        a = a.astype(np.float32)
        w[name] = W.bf16_round(a) if bf16 else a
    return cfg, w


def check(got, want, prec, what="", routed=False):
    """fp32: every row within 2e-4 of the largest logit.  bf16: within 4e-2, median row within
    1.5e-2; with routed experts a bf16 run may pick another expert than the float64 one where two
    scores nearly tie, which that row and (through state and cache) later ones then carry: there
    the bound holds for nine rows in ten and the median."""
    want = np.asarray(want).reshape(-1, np.asarray(want).shape[-1])
    got = np.asarray(got).reshape(want.shape)
    err = np.abs(got - want).max(axis=1) / np.abs(want).max()
    if prec == C.PREC_FP32:
        assert err.max() <= 2e-4, f"{what}: fp32 row error {err.max():.3e} at row {int(err.argmax())}"
        return
    bound = np.quantile(err, 0.9) if routed and len(err) >= 10 else err.max()
    if not (routed and len(err) < 10):
        assert bound <= 4e-2, f"{what}: bf16 row error {bound:.3e} (worst {err.max():.3e} at row {int(err.argmax())})"
    if len(err) >= 8:
        assert np.median(err) <= 1.5e-2, f"{what}: bf16 median row error {np.median(err):.3e}"


def setup(j, prec, seed=7, **kw):
    cfg, w = random_weights(j, seed, bf16=prec == C.PREC_BF16)
    return cfg, w, Engine(cfg, w, prec, **kw)


def no_close_calls(j, prec):
    """With random weights, some token in a few hundred has two expert scores closer than bf16
    rounding, and a run that then picks the other expert is no longer comparable from that token
    on (later layers, the state, the cache all carry it).  The bf16 runs of models with several
    layers therefore choose ALL experts of a layer (the scores still weight them); the choice among
    experts is tested in fp32 and, in bf16, on single layers."""
    if prec == C.PREC_FP32:
        return j
    j = copy.deepcopy(j)
    for lc in j["layers"]:
        if lc.get("mlp"):
            lc["mlp"]["router"]["top"] = lc["mlp"]["router"]["experts"]
    return j


def routed(j):
    return any(lc.get("mlp") for lc in j["layers"])


# ------------------------------------------------------------------ CPU: configuration
def test_config_reader_takes_every_size_from_the_file_and_the_tensor_shapes():
    j = mixed_model()
    cfg = C.ARCHITECTURES[j["architecture"]](j, shapes_of(j))
    assert cfg.arch == C.ARCH_LAZOVIK and not cfg.tied_head and cfg.needs_state_slots
    assert cfg.block_style == C.LBLOCK_SEQUENTIAL_PRENORM
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1, 4, 3)
    assert cfg.runs == (0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4)
    assert [l.mixer for l in cfg.layers] == [C.MIXER_GLA, C.MIXER_ATTN_TMIX, C.MIXER_GLA, C.MIXER_ATTN_TMIX, C.MIXER_GLA]
    a, b = cfg.layers[1], cfg.layers[3]
    assert (a.chunk, a.conv, a.rot_dims, a.lowrank, a.heads2, a.dim2) == (40, 3, 8, 8, 2, 16)
    assert a.rot_factor == 4.0 and a.rot_original == 64 and b.rot_factor == 0.0 and b.softcap == 30.0
    assert (b.kv_heads, b.top, b.experts, b.shared_ff, b.lowrank) == (1, 3, 9, 16, 5) and a.shared_ff == 0
    assert cfg.layers[2].mlp == C.MLP_NONE and cfg.layers[2].tau == 3.0 and cfg.layers[4].lowrank == 16
    sh = cfg.tensor_shapes()
    assert sh["loop.step"] == (3, 64) and sh["head"] == (211, 64) and "l2.norm2" not in sh
    assert sh["l1.mix.left.k.conv"] == (32, 3) and sh["l3.mix.right.u"] == (3, 8) and sh["l3.mlp.shared.sg"] == (1, 64)
    assert sh["l0.mix.a2"] == (48, 8) and "l1.mlp.shared.up" not in sh and sh["l3.mlp.e8.down"] == (64, 40)
    c, specs = cfg.to_c(C.PREC_FP32, num_state_slots=3)
    assert (c.loop_start, c.loop_stop, c.loop_times, c.num_state_slots) == (1, 4, 3, 3)
    assert specs[3].heads2 == 3 and specs[3].route_sigmoid == 1 and abs(specs[3].mix2_scale - 1.3) < 1e-6
    # no repeated run: the layers run once, in order
    assert C.lazovik_from_json(odd_model(), shapes_of(odd_model())).runs == (0, 1, 2)
    once = C.lazovik_from_json(model([layer(gla()), layer(gla())], loop=(1, 2, 1)), {"l0.mix.a1": (8, 64), "l1.mix.a1": (8, 64)})
    assert once.runs == (0, 1) and once.has_loop and once.tensor_shapes()["loop.step"] == (1, 64)
    with pytest.raises(ValueError):
        C.lazovik_from_json(model([dict(type="conv", mixer=gla()["mixer"], mlp=None)]), {})
    with pytest.raises(ValueError):  # the inner size of the decay projection is known from the checkpoint only
        C.lazovik_from_json(model([layer(gla())]), {})


def test_reference_mechanisms_against_hand_computed_values():
    """The restatement itself: a mask, a convolution, a scan and a shift small enough to check by hand."""
    assert ref.chunk_mask(5, 2).astype(int).tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 0, 1]]
    u = np.array([[1.0], [2.0], [4.0]])
    assert ref.short_conv(u, np.array([[10.0, 1.0]])).ravel().tolist() == [1.0, 12.0, 24.0]
    q = k = np.ones((2, 1)); v = np.array([[1.0], [3.0]]); d = np.full((2, 1), 0.5)
    assert ref.decayed_outer_product_scan(q, k, v, d).ravel().tolist() == [1.0, 3.5]
    assert ref.decayed_outer_product_scan(q, k, v, d, bonus=np.array([2.0])).ravel().tolist() == [2.0, 7.0]
    assert ref.token_shift(np.array([[2.0], [6.0]]), np.array([0.25])).ravel().tolist() == [1.5, 5.0]
    cos, sin = ref.rotation_tables({"dims": 4, "base": 100.0, "scaling": None}, 3)
    assert np.allclose(cos[2], [np.cos(2.0), np.cos(0.2)]) and np.allclose(sin[1], [np.sin(1.0), np.sin(0.1)])
    j = model([layer(gla(), moe())], loop=None)
    assert ref.execution_order(mixed_model())[4] == (1, 1) and ref.execution_order(j) == [(0, None)]


# ------------------------------------------------------------------ GPU: each mechanism alone
CASES = {
    "gla": lambda: [layer(gla())],
    "gla_wide": lambda: [layer(gla(heads=1, dim=200, vdim=40, tau=16.0, rank=12))],
    "attention_only": lambda: [layer(par(rs=0.0, chunk=19))],
    "time_mixing_only": lambda: [layer(par(ls=0.0))],
    "parallel": lambda: [layer(par(conv=4, chunk=33))],
    "no_rotation_scaling_no_cap": lambda: [layer(par(scaling=None, softcap=0.0, rot_dims=16))],
    "experts": lambda: [layer(gla(), moe(ff=32, experts=6, top=2, shared=0))],
    "experts_and_always_on": lambda: [layer(gla(), moe(ff=12, experts=4, top=4, shared=200))],
    "repeat": lambda: [layer(gla()), layer(par())],
    "repeat_once": lambda: [layer(par()), layer(gla())],  # one pass: still opened by the pass's vector
}
LOOPS = {"repeat": (0, 2, 3), "repeat_once": (1, 2, 1)}


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("case", sorted(CASES))
def test_each_mechanism_alone(case, prec):
    j = model(CASES[case](), loop=LOOPS.get(case))
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 90, 1)
        got, _ = eng.step([("a", toks, list(range(90)))])
        check(got, ref.forward(j, w, toks), prec, case, routed(j))
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("which", ["mixed", "odd", "mma"])
def test_prefill_equals_token_by_token_decoding(which, prec):
    j = no_close_calls({"mixed": mixed_model, "odd": odd_model, "mma": mma_model}[which](), prec)
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
def test_portions_of_several_sizes_down_to_two_tokens(prec):
    j = no_close_calls(mixed_model(), prec)
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 331, 3)
        want = ref.forward(j, w, toks)
        got, pos = [], 0
        # portions end inside chunks, on chunk borders (40, 80; 23, 46), and one crosses the page border at 256
        for n in [2, 3, 2, 16, 17, 40, 1, 5, 100, 2, 71, 2, 70]:
            out, _ = eng.step([("p", toks[pos:pos + n], list(range(n)))])
            got.append(out)
            pos += n
        assert pos == 331
        check(np.concatenate(got), want, prec, "portions", True)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_batches_of_unequal_requests_equal_each_alone(prec):
    j = no_close_calls(mma_model() if prec == C.PREC_BF16 else mixed_model(), prec)
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
        for r in range(5):  # 5 requests through 2 slots and 3 pages; each leaves state, tails and keys behind
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


# ------------------------------------------------------------------ GPU: chunk edges, far keys
BIG = 5


def make_standout(w, value_weights, gain):
    """The blocks norm their input, so a token cannot stand out by the size of its embedding.
    Instead: entry 0 of every embedding is zero except token BIG's, which is nothing else, and
    column 0 of the first layer's value projection is multiplied by `gain` — token BIG's value
    (and only its) is that much larger than any other."""
    w["embed"][:, 0] = 0.0
    w["embed"][BIG] = 0.0
    w["embed"][BIG, 0] = 8.0
    for name in value_weights:
        w[name][:, 0] *= gain
    return w


def edge_model(chunk, big_heads=False, conv=3, layers=1):
    """Attention only: the time-mixing side scaled by zero, no feed-forward.  (With a convolution
    of several taps a second layer would carry what position edge - 1 saw over the edge.)"""
    d = 64 if big_heads else 16
    mk = lambda: layer(par(heads=2, kv_heads=1, dim=d, vdim=d, conv=conv, chunk=chunk, rot_dims=8, rs=0.0, softcap=50.0))
    return model([mk() for _ in range(layers)], width=64)


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("chunk", [33, 64, 250])
def test_a_key_just_inside_and_just_outside_the_chunk_in_prompts_and_decoding(chunk, prec):
    """One token's value is 40 times the others' (make_standout), so it dominates whatever sees it.  It
    sits five places before a chunk's end: the last position of the chunk sees it, the first of
    the next chunk sees nothing of it (the convolution's reach has ended too).  A mask that is one
    position off changes those logits grossly, in bf16 too.  Probed inside a prompt (the chunk edge
    also near the page border), then with the same positions decoded."""
    j = edge_model(chunk, big_heads=prec == C.PREC_BF16)
    cfg, w = random_weights(j, 11, bf16=prec == C.PREC_BF16)
    big = BIG
    make_standout(w, ["l0.mix.left.v"], 40.0)
    eng = Engine(cfg, w, prec)
    try:
        for c in sorted({1, 256 // chunk, 256 // chunk + 1}):
            edge = c * chunk  # first position of a chunk
            place = edge - 5
            n = edge + 4
            toks = [t if t != big else 6 for t in prompt(j, n, 17 + c)]
            plain = ref.forward(j, w, toks)
            toks[place] = big
            want = ref.forward(j, w, toks)
            # the test's own premise: seen at edge - 1, gone without a trace at edge
            assert np.abs(want[edge - 1] - plain[edge - 1]).max() > 0.05 * np.abs(want).max()
            assert np.abs(want[edge:] - plain[edge:]).max() < 1e-9
            probes = [edge - 2, edge - 1, edge, edge + 1]
            got, _ = eng.step([("p", toks, probes)])
            check(got, want[probes], prec, f"prompt, edge {edge}")
            eng.end("p")
            eng.step([("d", toks[:edge - 3], [])])
            rows = [eng.step([("d", [toks[t]], [0])], decode=True)[0][0] for t in range(edge - 3, n)]
            check(np.stack(rows), want[edge - 3:], prec, f"decoded, edge {edge}")
            eng.end("d")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_a_far_key_among_hundreds_and_the_first_key_of_a_chunk(prec):
    """Attention only, one chunk of 600 positions from 300 on: the standout token at the chunk's
    first position (300) is read from 880, over two page borders; the one at 299 is not."""
    j = edge_model(300, big_heads=prec == C.PREC_BF16, conv=1, layers=2)
    cfg, w = random_weights(j, 14, bf16=prec == C.PREC_BF16)
    make_standout(w, ["l0.mix.left.v"], 400.0)
    eng = Engine(cfg, w, prec)
    try:
        base = [t if t != 5 else 6 for t in prompt(j, 599, 15)]
        inside, outside = list(base), list(base)
        inside[300] = 5
        outside[299] = 5
        plain, w_in, w_out = (ref.forward(j, w, t) for t in (base, inside, outside))
        assert np.abs(w_in[598] - plain[598]).max() > 0.05 * np.abs(plain).max()
        assert np.abs(w_out[300:] - plain[300:]).max() < 1e-9
        for toks, want, tag in ((inside, w_in, "inside"), (outside, w_out, "outside")):
            got, _ = eng.step([(tag, toks[:590], [300, 301, 589])])
            rows = [eng.step([(tag, [toks[t]], [0])], decode=True)[0][0] for t in range(590, 599)]
            check(np.concatenate([got, np.stack(rows)]), want[[300, 301, 589] + list(range(590, 599))], prec, tag)
            eng.end(tag)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("kind", ["gla", "time_mixing"])
def test_a_far_token_reaches_through_the_recurrent_state(kind, prec):
    """Recurrent layers only (the attention side scaled by zero): nothing but the carried state
    links position 600 to position 2.  The prompt goes in portions and then decodes, over two page borders."""
    if kind == "gla":
        j = model([layer(gla(heads=2, dim=64, vdim=16, tau=16.0)), layer(gla(heads=2, dim=32, vdim=32, tau=16.0))])
    else:
        j = model([layer(par(ls=0.0, heads2=2, dim2=32)), layer(par(ls=0.0, heads2=1, dim2=64))])
    cfg, w = random_weights(j, 12, bf16=prec == C.PREC_BF16)
    for name in w:  # slow decay: the state remembers
        if name.endswith("a2.b"):
            w[name][:] = 7.0
        if name.endswith(".w0"):
            w[name][:] = -7.0
        if name.endswith(".a2") or name.endswith(".w2"):
            w[name][:] *= 0.1
    make_standout(w, ["l0.mix.v" if kind == "gla" else "l0.mix.right.v"], 300.0)
    eng = Engine(cfg, w, prec)
    try:
        toks = [t if t != BIG else 8 for t in prompt(j, 640, 13)]
        with_far = list(toks)
        with_far[2] = BIG
        want, without = ref.forward(j, w, with_far), ref.forward(j, w, toks)
        assert np.abs(want[600:] - without[600:]).max() > 0.1 * np.abs(want[600:]).max()  # the test's own premise
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
@pytest.mark.parametrize("which,prec", [("odd", C.PREC_FP32), ("mixed", C.PREC_FP32), ("mixed", C.PREC_BF16), ("mma", C.PREC_BF16)])
def test_first_tokens_of_a_sequence(which, prec):
    """Positions 0, 1, 2: shorter than the convolution, the chunk and any tile; a one-token prompt;
    the token shift and the convolution read zeros before the start, whatever the slot held."""
    j = no_close_calls({"mixed": mixed_model, "odd": odd_model, "mma": mma_model}[which](), prec)
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


# ------------------------------------------------------------------ GPU: models drawn at random
def draw_model(rng):
    """Sizes, head counts, layer order, chunks, constants and the repeated run all drawn."""
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        if rng.random() < 0.5:
            mix = gla(heads=int(rng.integers(1, 7)), dim=int(rng.choice([8, 12, 16, 32, 48, 64, 96, 128])),
                      vdim=int(rng.choice([8, 16, 24, 32, 64, 96, 128])), tau=float(rng.uniform(1, 32)), rank=int(rng.integers(2, 33)))
        else:
            kv, g = int(rng.integers(1, 5)), int(rng.choice([1, 2, 3, 4, 6]))
            dim = int(rng.choice([8, 16, 32, 64, 128]))
            sc = None if rng.random() < 0.4 else {"factor": float(rng.uniform(1.5, 8)), "original": int(rng.integers(16, 4096)),
                                                  "fast": float(rng.uniform(4, 64)), "slow": float(rng.uniform(0.5, 2))}
            mix = par(heads=kv * g, kv_heads=kv, dim=dim, vdim=int(rng.choice([8, 16, 32, 64, 128])), conv=int(rng.integers(1, 6)),
                      chunk=int(rng.integers(1, 300)), rot_dims=int(rng.integers(1, dim // 2 + 1)) * 2,
                      base=float(rng.choice([100.0, 10000.0, 500000.0])), scaling=sc, scale=float(dim ** -0.5 * rng.uniform(0.5, 2)),
                      softcap=float(rng.choice([0.0, 5.0, 20.0, 50.0])), heads2=int(rng.integers(1, 5)),
                      dim2=int(rng.choice([8, 16, 32, 64, 128])), rank=int(rng.integers(2, 33)),
                      ls=float(rng.uniform(0.3, 1.5)), rs=float(rng.uniform(0.3, 1.5)))
        mlp = None
        if rng.random() < 0.8:
            e = int(rng.integers(2, 21))
            mlp = moe(ff=int(rng.integers(8, 100)), experts=e, top=int(rng.integers(1, min(4, e) + 1)),
                      shared=0 if rng.random() < 0.3 else int(rng.integers(8, 120)))
        layers.append(layer(mix, mlp))
    loop = None
    if rng.random() < 0.7:
        a = int(rng.integers(0, len(layers)))
        loop = (a, int(rng.integers(a + 1, len(layers) + 1)), int(rng.integers(1, 4)))
    return model(layers, vocab=int(rng.integers(50, 500)), width=int(rng.choice([64, 96, 128, 192, 256])),
                 eps=float(rng.choice([1e-5, 1e-6, 1e-4])), loop=loop)


@gpu
@pytest.mark.parametrize("seed", range(8))
def test_models_drawn_at_random(seed):
    """Whole prompt, then the same tokens in drawn portions with the last ones decoded, beside a
    second request that comes and goes; fp32, every row."""
    rng = np.random.default_rng(4000 + seed)
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


def strip_private(j):
    j = copy.deepcopy(j)
    for lc in j["layers"]:
        lc["mixer"].pop("_rank", None)
        if "right" in lc["mixer"]:
            lc["mixer"]["right"].pop("_rank", None)
    return j


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_command_line_on_a_model_directory(tmp_path, dtype):
    """bin/trace_run: config.json + model.safetensors (bf16) in, logits of the wanted places out;
    the sizes that only tensor shapes give come from the file's header."""
    j = no_close_calls(mixed_model(), C.PREC_FP32 if dtype == "float32" else C.PREC_BF16)
    cfg, w = random_weights(j, 22, bf16=True)
    mdir, out = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(strip_private(j)))
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
    j = model([layer(gla(heads=1, dim=300, vdim=8))])
    cfg, w = random_weights(j, 1)
    with pytest.raises(L.NvllmError):
        R.CudaModelRunner(cfg, w.items(), precision=C.PREC_FP32, num_kv_blocks=2, sampling=None, num_state_slots=1)
