"""The Zivitar design in the library against the plain implementation of `plain_zivitar.py`: small
configurations made here (sizes and options that differ from each other in every respect), random weights,
every comparison on logits.  CPU tests cover the configuration reader, the model description and the cache's
page rules; GPU tests cover the kernels and the engine."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zivitar as P
from helpers import BF16_TOL, FP32_TOL, ROOT, random_tokens, rel_err


def tol_for(dtype):
    """The float32 engine is held to the library's float32 bound.  In bfloat16 the models here are 32 to 96 wide
    and deep in roundings (norms, three to five products and two activations a layer, several layers, peaked
    attention), and rows are compared a few at a time: twice the library's bound; a key seen or missed by mistake
    moves these logits by 15 % and more (the tests on the window's edges show it)."""
    return FP32_TOL if dtype == "float32" else 2 * BF16_TOL


def attention(heads, kv_heads, dim, vdim, scale, diff, conv=None, mask=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff)
    if conv:
        m["conv"] = conv
    if mask:
        m["mask"] = dict(size=mask[0], keep_first=mask[1])
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return m


def layer(kind, mixer, ff=None, limit=None, weights_of=None):
    d = dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


ATT_A = attention(4, 2, 16, 24, 0.3, 0.4, conv=2, mask=(40, 3), rot=(8, 1000.0, (2.0, 64, 8.0, 1.0)))
# three streams, a layer used twice, a lightning layer without feed-forward, scale and soft cap on the logits
CFG_A = dict(architecture="Zivitar", vocab=160, width=64, norm=dict(eps=1e-5), streams=3, logit_scale=0.7, logit_softcap=8.0,
             layers=[layer("attention", ATT_A, 96, 2.0),
                     layer("lightning", dict(heads=2, dim=16, vdim=40, decay=[0.9, 0.999])),
                     layer("attention", ATT_A, 96, 2.0, weights_of=0),
                     layer("lightning", dict(heads=4, dim=8, vdim=16, decay=[0.5, 0.8, 0.95, 0.99]), 72, 0.5)])
# one residual stream without connections, no cap; attention without convolution, window or rotation; one with a
# window of just over a page that keeps more first keys than a page holds, four taps and whole vectors rotated
CFG_B = dict(architecture="Zivitar", vocab=200, width=96, norm=dict(eps=1e-6),
             layers=[layer("attention", attention(3, 3, 8, 32, 0.5, 0.25), 40, 1.0),
                     layer("lightning", dict(heads=1, dim=24, vdim=8, decay=[0.97]), 64, 3.0),
                     layer("attention", attention(6, 2, 24, 16, 0.2, 0.7, conv=4, mask=(65, 70), rot=(24, 50.0)))])
# a single stream that still has connections, one tap, a window smaller than the chunk the kernel walks in
CFG_C = dict(architecture="Zivitar", vocab=96, width=32, norm=dict(eps=1e-5), streams=1, logit_softcap=5.0,
             layers=[layer("attention", attention(2, 1, 8, 8, 0.35, 0.1, conv=1, mask=(5, 0), rot=(4, 100.0, (8.0, 16, 4.0, 1.0))), 48, 1.5),
                     layer("lightning", dict(heads=2, dim=4, vdim=16, decay=[1.0, 0.7]), 16, 0.8, ),
                     layer("lightning", dict(heads=2, dim=4, vdim=16, decay=[1.0, 0.7]), 16, 0.8, weights_of=1)])
# key and value sizes that the tensor-core prompt kernel takes: three query heads per key/value head with a window
# that is no multiple of anything, and one head per key/value head without a window
CFG_D = dict(architecture="Zivitar", vocab=128, width=64, norm=dict(eps=1e-5), streams=2, logit_scale=1.5,
             layers=[layer("attention", attention(6, 2, 32, 48, 0.2, 0.5, conv=3, mask=(37, 2), rot=(16, 300.0)), 64, 1.0),
                     layer("attention", attention(2, 2, 16, 64, 0.3, 0.2, rot=(16, 10000.0, (4.0, 32, 16.0, 1.0)))),
                     layer("lightning", dict(heads=2, dim=32, vdim=32, decay=[0.99, 0.9]), 32, 1.0)])
# widths that are multiples of nothing: the bfloat16 products run on zero-padded operands, loads are scalar
CFG_E = dict(architecture="Zivitar", vocab=75, width=36, norm=dict(eps=1e-5), streams=2,
             layers=[layer("attention", attention(2, 1, 10, 7, 0.3, 0.3, conv=3, mask=(33, 1), rot=(6, 100.0)), 22, 1.0),
                     layer("lightning", dict(heads=3, dim=5, vdim=9, decay=[0.9, 0.95, 0.99]), 13, 2.0)])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D, "E": CFG_E}


def sharpened(w, factor=4.0):
    """Attention made peaked, so that a key that is wrongly seen or missed moves the logits."""
    out = dict(w)
    for name in w:
        if name.endswith(".mix.q") or name.endswith(".mix.k"):
            out[name] = (w[name] * factor).to(torch.bfloat16).to(P.DT)
    return out


def folder(tmp_path, cfg, seed, sharpen=2.0):
    w = sharpened(P.random_weights(cfg, seed), sharpen)
    d = P.save_folder(cfg, w, str(tmp_path / f"model{seed}"))
    return d, w


# ------------------------------------------------------------------------------------------------
# without a device
# ------------------------------------------------------------------------------------------------
def test_the_plain_implementation_gives_the_same_logits_in_pieces():
    for name, cfg in CONFIGS.items():
        w = P.random_weights(cfg, 3)
        ids = random_tokens(90, cfg["vocab"], 7)
        whole = P.forward(cfg, w, ids)
        pieces = P.forward_in_pieces(cfg, w, ids, [1, 1, 2, 3, 60, 1, 22])
        assert float((whole - pieces).abs().max()) < 1e-9, name


def test_configuration_is_read_by_key_and_written_back():
    from janus_b200.config import ConfigError, resolve_architecture
    for cfg in CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        assert json.loads(json.dumps(c.to_dict())) == json.loads(json.dumps(cfg))
    arch = resolve_architecture(CFG_A)
    c = arch.config_class.from_dict(CFG_A)
    assert c.owner(2) == 0 and c.streams == 3 and c.layers[1].mlp is None
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 0, "mlp", "kind"), "routed", "kind"),
                              (("layers", 2, "weights_of"), 2, "weights_of"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mixer", "decay"), [0.5], "decay"), (("norm",), None, "norm"),
                              (("layers", 0, "mixer", "rot", "dims"), 7, "dims")):
        bad = copy.deepcopy(CFG_A)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            arch.config_class.from_dict(bad)
    # a layer that borrows tensors must have the sizes of the layer it borrows from
    bad = copy.deepcopy(CFG_A)
    bad["layers"][2]["mixer"] = dict(bad["layers"][2]["mixer"], vdim=32)
    with pytest.raises(ConfigError, match="differs"):
        arch.config_class.from_dict(bad)


def test_the_model_description_names_every_tensor_once_and_shares_borrowed_layers():
    from janus_b200.config import resolve_architecture
    from janus_b200.models.zivitar import zivitar_spec
    arch = resolve_architecture(CFG_A)
    c = arch.config_class.from_dict(CFG_A)
    spec = zivitar_spec(c)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 0, 2] and spec.residual_streams == 3
    names = {s.name: tuple(s.shape) for s in arch.weight_specs(c)}
    want = {k: tuple(v.shape) for k, v in P.random_weights(CFG_A, 0).items()}
    assert names == want
    assert "l1.hc2.in" not in names and "l2.norm1" not in names and names["l0.mix.q.conv"] == (4 * 2 * 16, 2)
    b = arch.config_class.from_dict(CFG_B)
    assert zivitar_spec(b).residual_streams == 1 and zivitar_spec(b).logit_transforms == ()
    assert all(l.arrangement == "pre_norm" for l in zivitar_spec(b).layers)
    assert set(P.random_weights(CFG_B, 0)) == {s.name for s in arch.weight_specs(b)}


def test_a_window_that_keeps_first_keys_keeps_their_pages_and_values_have_their_own_shape():
    from janus_b200.cache import PAGE_SIZE, SequenceCache
    from janus_b200.parts import KVSpec, StateSpec
    kv = KVSpec(4, 8, window=65, keep_first=70, n_value_heads=2, value_dim=24)
    cache = SequenceCache([(kv, StateSpec((3, 10))), None, StateSpec((2, 2))], 64 * 12, 3, torch.float32, torch.device("cpu"))
    g = cache.groups[0]
    assert tuple(g.k[0].shape[1:]) == (4, PAGE_SIZE, 8) and tuple(g.v[0].shape[1:]) == (2, PAGE_SIZE, 24)
    assert tuple(cache.states[0].shape) == (3, 3, 10) and tuple(cache.states[2].shape) == (3, 2, 2)
    s = cache.alloc_slot()
    cache.reserve(s, 400)
    cache.advance(s, 400)
    pages = g.pages[s]
    # keys 0..69 lie on pages 0 and 1; the next query (400) sees keys from 336 on: pages 2, 3, 4 are passed
    assert pages[0] >= 0 and pages[1] >= 0 and pages[2] == pages[3] == pages[4] == -1 and pages[5] >= 0
    cache.check()
    cache.states[0][s].fill_(1.0)
    cache.free_slot(s)
    assert g.pool.n_held == 0
    assert cache.alloc_slot() == s and float(cache.states[0][s].abs().sum()) == 0.0


def test_ramped_frequencies_follow_their_definition():
    from janus_b200.parts.rope import RampedRotaryEncoding
    for dims, base, scaling in ((8, 1000.0, dict(factor=2.0, original=64, fast=8.0, slow=1.0)), (24, 50.0, None),
                                (4, 100.0, dict(factor=8.0, original=16, fast=4.0, slow=1.0))):
        enc = RampedRotaryEncoding(dims, base, 300, scaling)
        f, m = P.rotary_frequencies(dims, base, scaling)
        pos = torch.arange(300, dtype=P.DT)
        want = torch.stack([torch.cos(pos[:, None] * f) * m, torch.sin(pos[:, None] * f) * m], dim=-1)
        assert float((enc.table.to(P.DT) - want).abs().max()) < 1e-6


# ------------------------------------------------------------------------------------------------
# on the device
# ------------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


def load(d, dtype, max_tokens=2048, **kw):
    import janus_b200
    return janus_b200.load(d, dtype=dtype, max_tokens=max_tokens, **kw)


@gpu
def test_stream_kernels_activation_and_cap_against_their_formulas():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(0)
    for S, H, T in ((3, 40, 7), (1, 64, 5), (8, 33, 3)):
        x = torch.randn(T, S * H, generator=g)
        a, b, M = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(S, S, generator=g)
        gamma, y = torch.randn(H, generator=g), torch.randn(T, H, generator=g)
        xs = x.to(P.DT).view(T, S, H)
        u = torch.einsum("s,tsh->th", a.to(P.DT), xs)
        out = torch.empty(T, H, device="cuda")
        clear = torch.ones(T, H, device="cuda")
        ops.streams_rmsnorm(x.cuda(), S, a.cuda(), gamma.cuda(), 1e-5, out, clear=clear)
        assert rel_err(out.cpu(), P.rms_norm(u, gamma.to(P.DT), 1e-5)) < 1e-5 and float(clear.abs().sum()) == 0.0
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
        out2 = torch.empty(2, H, device="cuda")
        ops.streams_rmsnorm(x.cuda(), S, None, gamma.cuda(), 1e-5, out2, row_index=rows)
        assert rel_err(out2.cpu(), P.rms_norm(xs.sum(1), gamma.to(P.DT), 1e-5)[[T - 1, 0]]) < 1e-5
        xd = x.cuda()
        ops.streams_mix(xd, y.cuda(), M.cuda(), b.cuda(), S)
        want = torch.einsum("sr,tsh->trh", M.to(P.DT), xs) + b.to(P.DT)[None, :, None] * y.to(P.DT)[:, None, :]
        assert rel_err(xd.cpu().view(T, S, H), want) < 1e-5
    gu = torch.randn(6, 50, generator=g) * 3
    act = torch.empty(6, 20, device="cuda")
    ops.clamped_glu(gu.cuda(), act, 30, 1.5, 1.702)
    gg, uu = torch.clamp(gu[:, :20].to(P.DT), max=1.5), torch.clamp(gu[:, 30:50].to(P.DT), -1.5, 1.5)
    assert rel_err(act.cpu(), gg * torch.sigmoid(1.702 * gg) * (uu + 1)) < 1e-5
    z = torch.randn(5, 33, generator=g) * 20
    zd = z.cuda()
    ops.scale_softcap(zd, 0.5, 6.0)
    assert rel_err(zd.cpu(), 6.0 * torch.tanh(z.to(P.DT) * 0.5 / 6.0)) < 1e-5


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompts_of_unequal_lengths_in_one_step(tmp_path, name, dtype):
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 11)
    model = load(d, dtype)
    seqs = [random_tokens(n, cfg["vocab"], 100 + n) for n in (150, 1, 67, 2, 64)]
    slots = [model.alloc_slot() for _ in seqs]
    out = model.step([StepEntry(s, ids, range(len(ids))) for s, ids in zip(slots, seqs)]).cpu()
    ref = torch.cat([P.forward(cfg, w, ids) for ids in seqs])
    assert rel_err(out, ref) < tol_for(dtype)
    if dtype == "float32":
        at = 0
        for ids in seqs:          # every sequence by itself, the single token too
            assert rel_err(out[at:at + len(ids)], ref[at:at + len(ids)]) < tol_for(dtype), (name, len(ids))
            at += len(ids)
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_portions_then_single_tokens_in_a_batch_and_slots_used_again(tmp_path, name, dtype):
    """Prompts cut into portions of 2 to 64 tokens, unequal requests in one batch, then one token each until the
    shorter ones have ended; afterwards other requests take the freed slots and pages.  Every row is compared
    with the whole sequence's logits from the plain implementation."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 12)
    tol = tol_for(dtype)
    model = load(d, dtype, max_tokens=64 * 9, max_slots=3)
    for round_no, lengths in enumerate(((140, 75, 20), (90, 130, 129))):
        seqs = [random_tokens(n, cfg["vocab"], 7 * round_no + n) for n in lengths]
        ref = [P.forward(cfg, w, ids) for ids in seqs]
        slots = [model.alloc_slot() for _ in seqs]
        at = [0, 0, 0]
        for portion in ((2, 3, 2), (62, 5, 3), (1, 40, 2), (17, 2, 2)):
            entries, spans = [], []
            for i, n in enumerate(portion):
                entries.append(StepEntry(slots[i], seqs[i][at[i]:at[i] + n], range(n)))
                spans.append((i, at[i], n))
                at[i] += n
            out = model.step(entries).cpu()
            row = 0
            for i, lo, n in spans:
                assert rel_err(out[row:row + n], ref[i][lo:lo + n]) < tol, (round_no, i, lo, n)
                row += n
        live = [0, 1, 2]
        while live:
            out = model.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in live]).cpu()
            for row, i in enumerate(live):
                assert rel_err(out[row:row + 1], ref[i][at[i]:at[i] + 1]) < tol, (round_no, i, at[i])
                at[i] += 1
            for i in [i for i in live if at[i] == len(seqs[i])]:
                model.free_slot(slots[i])
                live.remove(i)
        model.engine.cache.check()
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_first_keys(tmp_path, dtype):
    """One attention layer with peaked attention: the logits of the plain implementation with the window or the
    number of kept keys off by one differ clearly from the right ones at the rows compared, in prompts and in
    single tokens, so a key that is seen or missed by mistake would show."""
    from janus_b200.engine import StepEntry
    cfg = dict(architecture="Zivitar", vocab=120, width=64, norm=dict(eps=1e-5), streams=2,
               layers=[layer("attention", attention(2, 1, 16, 16, 0.5, 0.3, conv=3, mask=(70, 5), rot=(16, 10000.0)))])
    w = sharpened(P.random_weights(cfg, 5), 2.0)
    # one token whose keys are large: it sits on the last kept place and on the first that is not kept
    w["embed"][111] = 0.0
    w["embed"][111, 7] = 8.0
    w["l0.mix.k"][:, 7] = (w["l0.mix.k"][:, 7] * 3.0).to(torch.bfloat16).to(P.DT)
    d = P.save_folder(cfg, w, str(tmp_path / "edge"))
    ids = random_tokens(210, cfg["vocab"] - 10, 9)
    ids[4] = ids[5] = 111
    ref = P.forward(cfg, w, ids)
    rows = list(range(60, 210))
    for key, delta in (("size", -1), ("size", 1), ("keep_first", -1), ("keep_first", 1)):
        off = copy.deepcopy(cfg)
        off["layers"][0]["mixer"]["mask"][key] += delta
        assert rel_err(P.forward(off, w, ids)[rows], ref[rows]) > 5 * tol_for(dtype), (key, delta)
    model = load(d, dtype, max_tokens=512)
    s = model.alloc_slot()
    out = model.step([StepEntry(s, ids[:150], range(150))]).cpu()
    assert rel_err(out, ref[:150]) < tol_for(dtype)
    for t in range(150, 210):          # the window and the kept keys pass page borders while single tokens come
        out = model.step([StepEntry(s, [ids[t]], [0])]).cpu()
        assert rel_err(out, ref[t:t + 1]) < tol_for(dtype), t
    held = [p for p in model.engine.cache.groups[0].pages[s]]
    assert held[0] >= 0 and held[1] == -1 and held[3] >= 0      # the kept keys' page stays, a passed one is given back
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_reaches_through_the_lightning_state(tmp_path, dtype):
    """A head whose decay is 1 carries a token from hundreds of positions back: changing that one token changes
    the last logits of the plain implementation clearly, and the library follows both versions."""
    from janus_b200.engine import StepEntry
    cfg = dict(architecture="Zivitar", vocab=90, width=32, norm=dict(eps=1e-5),
               layers=[layer("lightning", dict(heads=2, dim=8, vdim=8, decay=[1.0, 0.5]))])
    w = P.random_weights(cfg, 6)
    # weights made so that the far token shows: tokens 5, 77 and 12 are one feature each; the first head's keys
    # answer to the features of 77 and 12 and are next to nothing for token 5, its queries answer to token 5
    for tok, feature in ((5, 0), (77, 1), (12, 2)):
        w["embed"][tok] = 0.0
        w["embed"][tok, feature] = 1.0
    w["l0.norm1"][:3] = 1.0
    w["l0.mix.k"][:8] = 0.0
    w["l0.mix.k"][:8, 0], w["l0.mix.k"][:8, 1], w["l0.mix.k"][:8, 2] = -2.0, 2.0, 1.0
    w["l0.mix.q"][:8] = 0.0
    w["l0.mix.q"][:8, 0] = 1.0
    d = P.save_folder(cfg, w, str(tmp_path / "far"))
    ids = [5] * 400
    ids[3] = 77
    other = list(ids)
    other[3] = 12
    ref, ref_other = P.forward(cfg, w, ids), P.forward(cfg, w, other)
    assert rel_err(ref_other[-5:], ref[-5:]) > 5 * tol_for(dtype)
    model = load(d, dtype, max_tokens=1024)
    for seq, want in ((ids, ref), (other, ref_other)):
        s = model.alloc_slot()
        out = model.step([StepEntry(s, seq[:395], [394])]).cpu()
        assert rel_err(out, want[394:395]) < tol_for(dtype)
        for t in range(395, 400):
            out = model.step([StepEntry(s, [seq[t]], [0])]).cpu()
            assert rel_err(out, want[t:t + 1]) < tol_for(dtype)
        model.free_slot(s)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(tmp_path, dtype):
    """A sequence that starts with a single token and grows by one for 200 steps (replayed CUDA graphs): the
    first tokens, page borders at 64 and 128, a window of 65 that keeps 70 first keys."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS["B"]
    d, w = folder(tmp_path, cfg, 13)
    ids = random_tokens(200, cfg["vocab"], 21)
    ref = P.forward(cfg, w, ids)
    model = load(d, dtype, max_tokens=256, max_slots=2)
    s = model.alloc_slot()
    got = [model.step([StepEntry(s, [t], [0])]).cpu() for t in ids]
    assert rel_err(torch.cat(got), ref) < tol_for(dtype)
    assert model.engine.graph_captures >= 1
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_the_scheduler(tmp_path, dtype):
    """`write_random_model` -> `load` -> `generate`: five prompts in batches of two; every generated token is the
    plain implementation's pick given the tokens before it."""
    import janus_b200
    from janus_b200.weights import write_random_model
    d = write_random_model(CFG_A, str(tmp_path / "gen"), seed=31, dtype="bfloat16", std=0.1, norm_std=0.05)
    cfg, w = P.read_folder(d)
    assert cfg["streams"] == 3 and abs(float(w["l0.hc1.mix"][1, 1]) - 1.0) < 0.3 and abs(float(w["l0.hc1.mix"][0, 1])) < 0.3
    model = janus_b200.load(d, dtype=dtype, max_tokens=1024, max_slots=4)
    prompts = [random_tokens(n, cfg["vocab"], 3 + n) for n in (5, 70, 1, 33, 12)]
    out, stats = model.generate(prompts, max_tokens=10, batch_size=2)
    assert stats.batches == 3
    for p, o in zip(prompts, out):
        assert len(o) == 10
        logits = P.forward(cfg, w, list(p) + list(o))
        for j, tok in enumerate(o):
            row = logits[len(p) - 1 + j]
            slack = 1e-4 if dtype == "float32" else BF16_TOL
            assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), (p, j)


@gpu
def test_the_replay_program_serves_the_design(tmp_path):
    d, w = folder(tmp_path, CFG_C, 14)
    ids = random_tokens(40, CFG_C["vocab"], 2)
    steps = [dict(step=0, entries=[dict(id="x", tokens=ids[:30], want=[0, 29])], end=[])]
    steps += [dict(step=j + 1, entries=[dict(id="x", tokens=[ids[30 + j]], want=[0])], end=["x"] if j == 9 else [])
              for j in range(10)]
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "128"],
                         input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    got = np.concatenate([np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, CFG_C["vocab"]) for s in steps])
    ref = P.forward(CFG_C, w, ids)
    assert rel_err(got, ref[[0] + list(range(29, 40))]) < FP32_TOL


@gpu
def test_the_command_line_samples_from_the_design(tmp_path):
    """`python -m janus_b200 DIR ...`: greedy tokens equal those of `generate`, and sampling with a temperature, top-k
    and a seed runs through the device sampler; a folder with config.json alone runs with `--random-weights`."""
    d, w = folder(tmp_path, CFG_D, 15)
    base = [sys.executable, "-m", "janus_b200", d, "3,1,4,1,5", "9,2,6", "--max-tokens", "7", "--dtype", "float32", "--json"]
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.environ.get("PYTHONPATH", "")]))
    res = subprocess.run(base, capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    greedy = json.loads(res.stdout.strip().splitlines()[-1])["tokens"]
    for p, o in zip(([3, 1, 4, 1, 5], [9, 2, 6]), greedy):
        assert len(o) == 7
        logits = P.forward(CFG_D, w, p + o)
        assert all(int(logits[len(p) - 1 + j].argmax()) == tok for j, tok in enumerate(o))
    res = subprocess.run(base + ["--temperature", "0.9", "--top-k", "12", "--top-p", "0.9", "--seed", "4"],
                         capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    sampled = json.loads(res.stdout.strip().splitlines()[-1])["tokens"]
    assert [len(o) for o in sampled] == [7, 7] and all(0 <= t < CFG_D["vocab"] for o in sampled for t in o)
    only_config = tmp_path / "only_config"
    only_config.mkdir()
    (only_config / "config.json").write_text(json.dumps(CFG_A))
    res = subprocess.run([sys.executable, "-m", "janus_b200", str(only_config), "1,2,3", "--max-tokens", "4", "--random-weights",
                          "--json"], capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    assert len(json.loads(res.stdout.strip().splitlines()[-1])["tokens"][0]) == 4
