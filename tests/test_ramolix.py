"""The Ramolix design in the library against the plain implementation of `plain_ramolix.py`: small
configurations made here (sizes and options that differ from each other in every respect), random weights,
every comparison on logits or on a kernel's own output.  CPU tests cover the configuration reader, the model
description, the frequencies and the cache's rules; GPU tests cover each kernel alone, each mixer alone, and the
engine: whole prompts, portions, batches, slots and pages used again, windows' edges, far keys, long decoding,
generation, the replay program and the command line."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_ramolix as P
from helpers import BF16_TOL, FP32_TOL, ROOT, random_tokens, rel_err


def tol_for(dtype):
    """For a few rows that a test singles out, where a fault would move the logits by 0.4 of their range and more."""
    return FP32_TOL if dtype == "float32" else 0.15


class Rows:
    """Rows of logits against the plain implementation's.  The float32 engine is held, row by row and at once, to
    the library's float32 bound: every fault of the cache, the state, the batch or a kernel's indexing shows there.
    In bfloat16 the models here are 32 to 96 wide, every sublayer's output is divided by its root mean square
    (which makes a rounding error as large as the output is small after cancellation), and attention is peaked:
    a few rows in a hundred move by a tenth of the logits' range and more from rounding alone (a state-space
    head of a handful of state rows whose output nearly cancels is normed back to full size; the recurrence runs
    the same float32 kernels in both engines).  So the rows are judged together when a test ends: half of them
    within the library's bfloat16 bound, nine in ten within twice that, none off by the logits' whole range.  The
    rows that a fault would concern are singled out and held to a bound of their own by the tests on the window's
    edges, on far keys and on the first tokens."""

    def __init__(self, dtype):
        self.dtype, self.errors = dtype, []

    def add(self, out, ref, where=None):
        out, ref = np.asarray(out, dtype=np.float64), np.asarray(ref, dtype=np.float64)
        assert out.shape == ref.shape, f"shape {out.shape} != {ref.shape}"
        assert np.isfinite(out).all(), "non-finite values in the engine's output"
        e = np.abs(out - ref).max(axis=1) / (np.abs(ref).max() + 1e-12)
        if self.dtype == "float32":
            assert float(e.max()) < FP32_TOL, where
        self.errors.extend(e.tolist())

    def close(self):
        e = np.asarray(self.errors)
        assert e.size > 0
        if self.dtype != "float32":
            assert float(np.median(e)) < BF16_TOL and float((e > 2 * BF16_TOL).mean()) <= 0.1 and float(e.max()) < 1.0, \
                (float(np.median(e)), float((e > 2 * BF16_TOL).mean()), float(e.max()))


def attention(heads, kv_heads, dim, scale, mask=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if mask:
        m["mask"] = dict(size=mask)
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    return m


def latent(heads, dim, vdim, rank, scale, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=rank, scale=scale)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def config(vocab, width, eps, scale, mult, layers):
    return dict(architecture="Ramolix", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=scale),
                residual_mult=mult, layers=layers)


# two kv heads under a window shorter than a page with scaled, partial rotation; two latent layers of which the
# second borrows the first one's latents with other heads and sizes; a state-space layer without feed-forward
CFG_A = config(160, 64, 1e-5, 3.0, 0.6, [
    layer("attention", attention(4, 2, 16, 0.3, mask=40, rot=(8, 1000.0, (2.0, 1.0, 8.0, 64))), 96),
    layer("latent_attention", latent(2, 8, 24, 16, 0.4), 48),
    layer("mamba2", mamba(4, 8, 16, 2, 4, 2)),
    layer("latent_attention", latent(4, 16, 8, 16, 0.25, kv_from=1), 40),
    layer("mamba2", mamba(2, 24, 8, 1, 2, 1), 72)])
# attention without window or rotation, and one with a window of just over a page and whole heads rotated; a
# state-space layer whose groups are its heads, with a single tap; a multiplier of one
CFG_B = config(200, 96, 1e-6, 1.0, 1.0, [
    layer("mamba2", mamba(3, 16, 24, 3, 1, 3), 40),
    layer("attention", attention(3, 3, 8, 0.5), 64),
    layer("latent_attention", latent(3, 24, 16, 40, 0.2)),
    layer("attention", attention(6, 2, 24, 0.2, mask=65, rot=(24, 50.0)), 80)])
# a window smaller than the chunk the kernels walk in, a latent that three layers share, five taps
CFG_C = config(96, 32, 1e-5, 0.5, 1.7, [
    layer("latent_attention", latent(1, 8, 8, 8, 0.35), 48),
    layer("attention", attention(2, 1, 8, 0.35, mask=5, rot=(4, 100.0, (8.0, 1.0, 4.0, 16))), 16),
    layer("latent_attention", latent(2, 4, 16, 8, 0.5, kv_from=0)),
    layer("mamba2", mamba(2, 16, 12, 2, 5, 2), 16),
    layer("latent_attention", latent(3, 8, 4, 8, 0.3, kv_from=0), 24)])
# sizes that the tensor-core prompt kernels take, a window that is no multiple of anything, long state rows
CFG_D = config(128, 64, 1e-5, 8.0, 0.8, [
    layer("attention", attention(6, 2, 32, 0.2, mask=37, rot=(16, 300.0)), 64),
    layer("mamba2", mamba(2, 32, 80, 1, 3, 2), 32),
    layer("latent_attention", latent(4, 16, 32, 64, 0.3), 64),
    layer("attention", attention(2, 2, 64, 0.12, rot=(32, 10000.0, (4.0, 1.0, 16.0, 32))))])
# sizes that are multiples of nothing: the bfloat16 products run on zero-padded operands, heads and latents are
# stored with zero columns up to a size the bfloat16 attention kernels take, loads are scalar
CFG_E = config(75, 36, 1e-5, 2.5, 0.9, [
    layer("attention", attention(2, 1, 12, 0.3, mask=33, rot=(6, 100.0)), 22),
    layer("mamba2", mamba(3, 5, 7, 1, 3, 3), 13),
    layer("latent_attention", latent(3, 5, 9, 21, 0.3), 27),
    layer("latent_attention", latent(2, 7, 3, 21, 0.4, kv_from=2))])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D, "E": CFG_E}


def sharpened(w, factor=3.0):
    """Attention made peaked, so that a key that is wrongly seen or missed moves the logits."""
    out = dict(w)
    for name in w:
        if name.endswith(".mix.q") or name.endswith(".mix.q.norm"):
            out[name] = (w[name] * factor).to(torch.bfloat16).to(P.DT)
    return out


def folder(tmp_path, cfg, seed, sharpen=3.0):
    w = sharpened(P.random_weights(cfg, seed), sharpen)
    return P.save_folder(cfg, w, str(tmp_path / f"model{seed}")), w


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
    assert c.layers[3].mixer.kv_from == 1 and c.layers[2].mlp is None and c.residual_mult == 0.6
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 0, "mlp", "kind"), "routed", "kind"),
                              (("layers", 3, "mixer", "kv_from"), 3, "kv_from"), (("layers", 3, "mixer", "kv_from"), 2, "kv_from"),
                              (("layers", 3, "mixer", "kv_rank"), 24, "kv_rank"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 0, "mixer", "vdim"), 24, "vdim"), (("layers", 2, "mixer", "groups"), 3, "groups"),
                              (("layers", 2, "mixer", "norm_groups"), 5, "norm_groups"), (("norm",), None, "norm"),
                              (("embedding",), None, "embedding"), (("layers", 0, "mixer", "rot", "dims"), 7, "dims")):
        bad = copy.deepcopy(CFG_A)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            arch.config_class.from_dict(bad)


def test_the_model_description_names_every_tensor_once_and_borrowed_latents_are_places_that_read():
    from janus_b200.config import resolve_architecture
    from janus_b200.models.ramolix import ramolix_spec
    for cfg in CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        names = {s.name: tuple(s.shape) for s in arch.weight_specs(c)}
        assert names == {k: tuple(v.shape) for k, v in P.random_weights(cfg, 0).items()}
    c = resolve_architecture(CFG_C).config_class.from_dict(CFG_C)
    spec = ramolix_spec(c)
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, 0, None, 0]
    assert spec.head_weight is None and all(ls.arrangement == "output_norm" for ls in spec.layers)
    assert dict(spec.layers[0].arrangement_params) == {"residual_mult": 1.7} and spec.layers[2].feed_forward is None
    names = {s.name for s in resolve_architecture(CFG_C).weight_specs(c)}
    assert "l2.mix.dkv" not in names and "l0.mix.dkv.norm" in names and "l2.norm2" not in names


def test_band_scaled_frequencies_follow_their_definition():
    from janus_b200.parts.rope import BandScaledRotaryEncoding
    for dims, base, scaling in ((8, 1000.0, dict(factor=2.0, low=1.0, high=8.0, original=64)), (24, 50.0, None),
                                (4, 100.0, dict(factor=8.0, low=1.0, high=4.0, original=16)),
                                (32, 10000.0, dict(factor=4.0, low=1.0, high=8.0, original=256))):
        enc = BandScaledRotaryEncoding(dims, base, 300, scaling)
        f = P.rotary_frequencies(dims, base, scaling)
        pos = torch.arange(300, dtype=P.DT)
        want = torch.stack([torch.cos(pos[:, None] * f), torch.sin(pos[:, None] * f)], dim=-1)
        assert float((enc.table.to(P.DT) - want).abs().max()) < 1e-6
    # all three bands occur in the scaled cases above
    f0, f1 = P.rotary_frequencies(32, 10000.0, None), P.rotary_frequencies(32, 10000.0, dict(factor=4.0, low=1.0, high=8.0, original=256))
    ratio = (f1 / f0).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-12 and any(0.26 < r < 0.99 for r in ratio)


def test_a_place_whose_values_are_its_keys_has_one_set_of_pages_and_states_start_at_zero():
    from janus_b200.cache import PAGE_SIZE, SequenceCache
    from janus_b200.parts import KVSpec, StateSpec
    specs = [KVSpec(1, 24, values_are_keys=True), None, StateSpec((50,)), KVSpec(2, 8, window=40)]
    cache = SequenceCache(specs, 64 * 8, 3, torch.float32, torch.device("cpu"))
    latent_group = cache.groups[cache.group_of_place[0]]
    assert latent_group.v[0] is latent_group.k[0] and tuple(latent_group.k[0].shape[1:]) == (1, PAGE_SIZE, 24)
    window_group = cache.groups[cache.group_of_place[3]]
    assert window_group.v[3] is not window_group.k[3]
    s = cache.alloc_slot()
    cache.reserve(s, 200)
    cache.advance(s, 200)
    # the next query (200) sees keys from 161 on: pages 0 and 1 are passed in the window group only
    assert window_group.pages[s][0] == window_group.pages[s][1] == -1 and window_group.pages[s][2] >= 0
    assert all(p >= 0 for p in latent_group.pages[s])
    cache.states[2][s].fill_(1.0)
    cache.free_slot(s)
    cache.check()
    assert cache.alloc_slot() == s and float(cache.states[2][s].abs().sum()) == 0.0


# ------------------------------------------------------------------------------------------------
# on the device: every kernel alone
# ------------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


def load(d, dtype, max_tokens=2048, **kw):
    import janus_b200
    return janus_b200.load(d, dtype=dtype, max_tokens=max_tokens, **kw)


def dev(t, dtype=torch.float32):
    return t.to(dtype).cuda().contiguous()


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


@gpu
def test_output_norm_sum_and_the_gelu_gate_against_their_formulas():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(0)
    for T, H, mult in ((7, 40, 0.6), (3, 33, 1.0), (5, 2048, 1.7), (2, 4100, 0.5), (2, 8200, 1.1)):
        res, y, gamma = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g) * 3, torch.randn(H, generator=g)
        want = res.to(P.DT) + mult * P.rms_norm(y.to(P.DT), gamma.to(P.DT), 1e-5)
        for out_dtype in (torch.float32, torch.bfloat16):
            rd, yd = dev(res), dev(y)
            x = torch.empty(T, H, dtype=out_dtype, device="cuda")
            clear, clear2 = torch.ones(8, 4, device="cuda"), torch.ones(3, 12, device="cuda")
            ops.sublayer_norm_add(yd, dev(gamma), 1e-5, mult, rd, x, clear, clear2)
            assert rel_err(rd.cpu(), want) < 1e-5 and float(yd.abs().sum()) == 0.0
            assert float(clear.abs().sum()) == 0.0 and float(clear2.abs().sum()) == 0.0
            assert rel_err(x.float().cpu(), want) < (1e-5 if out_dtype == torch.float32 else 5e-3)
        rd, yd = dev(res), dev(y)
        ops.sublayer_norm_add(yd, dev(gamma, torch.bfloat16), 1e-5, mult, rd, None)         # the sum alone
        assert rel_err(rd.cpu(), res.to(P.DT) + mult * P.rms_norm(y.to(P.DT), gamma.to(torch.bfloat16).to(P.DT), 1e-5)) < 1e-5
        x = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        ops.sublayer_norm_add(None, None, 0.0, 0.0, rd, x)                                  # the cast alone
        assert torch.equal(x.cpu(), rd.cpu().to(torch.bfloat16))
    for H in (40, 33):                  # the embedding's scale in the gather's own launch
        table = torch.randn(20, H, generator=g).to(torch.bfloat16)
        out = torch.empty(4, H, device="cuda")
        ops.embed_gather(table.cuda(), i32([3, 19, 0, 3]), out, scale=2.5)
        assert rel_err(out.cpu(), table[[3, 19, 0, 3]].to(P.DT) * 2.5) < 1e-6
    gu = torch.randn(6, 50, generator=g) * 3
    act = torch.empty(6, 20, device="cuda")
    ops.clamped_glu(dev(gu), act, 30, ops.GELU_TANH_GATE, 1.0)
    assert rel_err(act.cpu(), P.gelu_tanh(gu[:, :20].to(P.DT)) * gu[:, 30:50].to(P.DT)) < 1e-5


@gpu
def test_the_gelu_gate_in_the_tensor_core_products_epilogue():
    from janus_b200.parts.linear import GatedLinear
    from janus_b200.engine.workspace import Workspace
    from janus_b200.kernels import ops

    class Ctx:
        workspace = Workspace(torch.device("cuda"))
    g = torch.Generator().manual_seed(1)
    for T, K, I in ((5, 64, 200), (100, 72, 130), (300, 128, 384)):     # decode-sized, a short prompt, CTA pairs
        x = (torch.randn(T, K, generator=g)).to(torch.bfloat16)
        wg, wu = (torch.randn(I, K, generator=g) * K ** -0.5).to(torch.bfloat16), (torch.randn(I, K, generator=g) * K ** -0.5).to(torch.bfloat16)
        lin = GatedLinear(K, I, torch.bfloat16, torch.device("cuda"), limit=ops.GELU_TANH_GATE)
        lin.load(wg, wu)
        out = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
        lin.forward(x.cuda(), out, Ctx)
        want = P.gelu_tanh(x.to(P.DT) @ wg.to(P.DT).T) * (x.to(P.DT) @ wu.to(P.DT).T)
        assert rel_err(out.float().cpu(), want) < 1e-2, (T, K, I)
    ops.check_kernel_status(torch.device("cuda"))


@gpu
def test_query_and_key_preparation_against_the_plain_mixer():
    """Bias, the value rows, one norm over all heads, partial rotation at each token's own position, pages."""
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    for H, G, d, rot, scaling in ((4, 2, 16, 8, dict(factor=2.0, low=1.0, high=8.0, original=64)), (3, 3, 10, 10, None),
                                  (2, 1, 24, 0, None)):
        T, page = 9, 64
        proj = torch.randn(T, (H + G) * d + 3, generator=g)
        bq, bk = torch.randn(H * d, generator=g), torch.randn(G * d, generator=g)
        wq, wk = torch.randn(H * d, generator=g), torch.randn(G * d, generator=g)
        positions = [0, 1, 2, 70, 71, 5, 300, 64, 63]
        rows = [3 * page + 5, 0, 1, 2 * page + 63, 4 * page, 77, 78, 200, 201]       # where each token's key goes
        rd = dict(dims=rot, base=100.0, scaling=scaling) if rot else None
        q = (proj[:, :H * d] + bq).to(P.DT)
        k = (proj[:, H * d:(H + G) * d] + bk).to(P.DT)
        pos = torch.tensor(positions)
        want_q = P.rotate(P.rms_norm(q, wq.to(P.DT), 1e-5).reshape(T, H, d), pos, rd).reshape(T, H * d)
        want_k = P.rotate(P.rms_norm(k, wk.to(P.DT), 1e-5).reshape(T, G, d), pos, rd)
        table = None
        if rot:
            f = P.rotary_frequencies(rot, 100.0, scaling)
            a = torch.arange(400, dtype=P.DT)[:, None] * f
            table = dev(torch.stack([torch.cos(a), torch.sin(a)], dim=-1))
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            kc = torch.zeros(6, G, page, d, dtype=dtype, device="cuda")
            vc = torch.zeros_like(kc)
            qo = torch.empty(T, H * d, dtype=dtype, device="cuda")
            ops.qk_norm_rope_cache(dev(proj), dev(bq), dev(bk), dev(wq), dev(wk), 1e-5, table, rot, i32(positions), qo,
                                   i32(rows), kc, vc, H, G, d, page)
            assert rel_err(qo.float().cpu(), want_q) < tol
            got_k = torch.stack([kc[r // page, :, r % page].float().cpu() for r in rows])
            got_v = torch.stack([vc[r // page, :, r % page].float().cpu() for r in rows])
            assert rel_err(got_k, want_k) < tol and rel_err(got_v, k.reshape(T, G, d)) < tol
            assert int((kc != 0).any(dim=-1).sum()) == T * G          # no other row was touched
            q2 = torch.empty_like(qo)
            ops.qk_norm_rope_cache(dev(proj[:, :H * d]), dev(bq), None, dev(wq), None, 1e-5, table, rot, i32(positions), q2,
                                   None, None, None, H, G, d, page, write_kv=False)
            assert torch.equal(q2, qo)
            # heads stored wider than they are: the same numbers, zeros behind them
            dp = d + 6
            kc, vc = torch.zeros(6, G, page, dp, dtype=dtype, device="cuda"), torch.zeros(6, G, page, dp, dtype=dtype, device="cuda")
            q3 = torch.full((T, H * dp), 7.0, dtype=dtype, device="cuda")
            ops.qk_norm_rope_cache(dev(proj), dev(bq), dev(bk), dev(wq), dev(wk), 1e-5, table, rot, i32(positions), q3,
                                   i32(rows), kc, vc, H, G, d, page, stored_dim=dp)
            q3 = q3.view(T, H, dp)
            assert torch.equal(q3[:, :, :d].reshape(T, H * d), qo) and float(q3[:, :, d:].abs().sum()) == 0.0
            assert rel_err(torch.stack([kc[r // page, :, r % page, :d].float().cpu() for r in rows]), want_k) < tol
            assert float(kc[..., d:].abs().sum()) == 0.0 and float(vc[..., d:].abs().sum()) == 0.0


@gpu
def test_latent_preparation_against_its_formula():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    for Q, r in ((48, 16), (15, 24), (512, 7)):
        T, page = 6, 64
        proj, w = torch.randn(T, Q + r + 2, generator=g), torch.randn(r, generator=g)
        rows = [5, 64, 63, 130, 0, 300]
        want = P.rms_norm(proj[:, Q:Q + r].to(P.DT), w.to(P.DT), 1e-6)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            cache = torch.zeros(5, 1, page, r, dtype=dtype, device="cuda")
            qo = torch.empty(T, Q, dtype=dtype, device="cuda")
            ops.latent_prep(dev(proj), Q, r, dev(w), 1e-6, qo, i32(rows), cache)
            assert rel_err(qo.float().cpu(), proj[:, :Q]) < tol
            assert rel_err(torch.stack([cache[x // page, 0, x % page].float().cpu() for x in rows]), want) < tol
            assert int((cache != 0).any(dim=-1).sum()) == T
            wide = torch.zeros(5, 1, page, r + 3, dtype=dtype, device="cuda")
            ops.latent_prep(dev(proj), Q, r, dev(w), 1e-6, qo, i32(rows), wide, stored_rank=r + 3)
            assert torch.equal(wide[..., :r], cache) and float(wide[..., r:].abs().sum()) == 0.0


def plain_conv(u, w, b, before):
    taps = w.shape[1]
    padded = torch.cat([before, u])
    out = sum(padded[j:j + u.shape[0]] * w[:, j] for j in range(taps))
    return P.silu(out + b), padded[padded.shape[0] - (taps - 1):]


@gpu
def test_the_short_convolution_with_its_state_in_portions_down_to_one_token():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    for C, taps, col0, pad, off in ((20, 4, 3, 8, 11), (7, 2, 3, 8, 11), (130, 1, 3, 8, 11), (33, 5, 3, 8, 11),
                                    (24, 4, 4, 8, 12), (520, 3, 8, 4, 0), (16, 8, 0, 0, 4), (12, 1, 4, 4, 8)):
        ld = col0 + C + pad       # the last four: whole 16-byte vectors everywhere, prompt steps take the vector kernel
        w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
        state = torch.zeros(4, off + (taps - 1) * C + (2 if pad == 8 else 4), device="cuda")
        slots = [2, 0]
        seqs = [torch.randn(140, ld, generator=g), torch.randn(125, ld, generator=g)]
        before = [torch.zeros(taps - 1, C, dtype=P.DT) for _ in seqs]
        at = [0, 0]
        for portion in ((1, 2), (1, 1), (1, 1), (2, 1), (3, 17), (30, 1), (1, 1), (1, 1), (33, 70), (2, 29), (65, 1)):
            xs = [s[a:a + n] for s, a, n in zip(seqs, at, portion)]
            proj = torch.cat(xs)
            T = proj.shape[0]
            out = torch.empty(T, C, device="cuda")
            ops.causal_conv_silu(dev(proj), col0, C, dev(w), dev(b), taps, state, off, i32([0] * portion[0] + [1] * portion[1]),
                                 i32([0, portion[0], T]), i32(slots), out, 2, single_tokens=portion == (1, 1))
            want = []
            for i, x in enumerate(xs):
                y, before[i] = plain_conv(x[:, col0:col0 + C].to(P.DT), w.to(P.DT), b.to(P.DT), before[i])
                want.append(y)
                at[i] += portion[i]
                if taps > 1:
                    got_state = state[slots[i], off:off + (taps - 1) * C].view(taps - 1, C).cpu()
                    assert rel_err(got_state, before[i]) < 1e-6, (C, taps, portion)
            assert rel_err(out.cpu(), torch.cat(want)) < 1e-5, (C, taps, portion)
        assert float(state[:, :off].abs().sum()) == 0.0 and float(state[1].abs().sum()) == 0.0


def plain_scan(x, B, C, dt_raw, dt_bias, A_log, D, S):
    """x [T, H, P], B and C [T, G, N], dt_raw [T, H], S [H, N, P] -> (y [T, H, P], S)"""
    T, H, Pv = x.shape
    G = B.shape[1]
    dt = P.softplus(dt_raw + dt_bias)
    y = torch.zeros_like(x)
    S = S.clone()
    for t in range(T):
        for h in range(H):
            gidx = h // (H // G)
            S[h] = torch.exp(-torch.exp(A_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, gidx], x[t, h])
            y[t, h] = S[h].T @ C[t, gidx] + D[h] * x[t, h]
    return y, S


@gpu
def test_the_recurrence_whole_in_segments_and_token_by_token():
    """Sequences of unequal lengths in one launch; a long one runs in segments (three passes) and must agree with
    the walk in one piece; then single tokens continue from the state that was left."""
    from janus_b200.engine.workspace import Workspace
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    ws = Workspace(torch.device("cuda"))
    for H, G, N, Pv in ((4, 2, 16, 8), (3, 1, 7, 5), (2, 2, 80, 70), (1, 1, 200, 3)):
        lens = (300, 1, 37)
        off, total = 5, 5 + H * N * Pv + 3
        ld = H * Pv + 2 * G * N + 4
        state = torch.zeros(5, total, device="cuda")
        slots = [3, 1, 4]
        dt_bias, A_log, D = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) * 0.5 - 1.0, torch.randn(H, generator=g)
        S = [torch.zeros(H, N, Pv, dtype=P.DT) for _ in lens]

        def run(xbc, dt_raw, q_lens, use_ws):
            T = xbc.shape[0]
            out = torch.empty(T, H * Pv, device="cuda")
            starts = np.concatenate([[0], np.cumsum(q_lens)]).tolist()
            ops.mamba2_scan(dev(xbc), H * Pv, H * Pv + G * N, dev(dt_raw), dev(dt_bias), dev(A_log), dev(D), out, state, off,
                            i32(starts), i32(slots), len(q_lens), H, G, N, Pv, max(q_lens), ws if use_ws else None)
            return out.cpu()

        def plain(xbc, dt_raw, q_lens):
            outs, at = [], 0
            for i, n in enumerate(q_lens):
                seg = xbc[at:at + n].to(P.DT)
                y, S[i] = plain_scan(seg[:, :H * Pv].reshape(n, H, Pv), seg[:, H * Pv:H * Pv + G * N].reshape(n, G, N),
                                     seg[:, H * Pv + G * N:H * Pv + 2 * G * N].reshape(n, G, N), dt_raw[at:at + n].to(P.DT),
                                     dt_bias.to(P.DT), A_log.to(P.DT), D.to(P.DT), S[i])
                outs.append(y.reshape(n, H * Pv))
                at += n
            return torch.cat(outs)

        xbc, dt_raw = torch.randn(sum(lens), ld, generator=g), torch.randn(sum(lens), H, generator=g)
        want = plain(xbc, dt_raw, lens)
        segmented = run(xbc, dt_raw, lens, True)
        after_segments = state.clone()
        state.zero_()
        whole = run(xbc, dt_raw, lens, False)
        assert rel_err(segmented, want) < 2e-5 and rel_err(whole, want) < 2e-5, (H, G, N, Pv)
        assert rel_err(after_segments.cpu(), state.cpu()) < 2e-5
        for i, s in enumerate(slots):
            assert rel_err(state[s, off:off + H * N * Pv].cpu().view(H, N, Pv), S[i]) < 2e-5
        assert float(state[:, :off].abs().sum()) == 0.0 and float(state[0].abs().sum()) == 0.0
        for _ in range(3):                               # one token each, from the state that was left
            xbc, dt_raw = torch.randn(3, ld, generator=g), torch.randn(3, H, generator=g)
            assert rel_err(run(xbc, dt_raw, (1, 1, 1), True), plain(xbc, dt_raw, (1, 1, 1))) < 2e-5
    # large step sizes and strongly negative ones (softplus has no clamp), with decays from next to one down to
    # nothing at all: the late decays are rescaled in time, nothing over- or underflows
    H, G, N, Pv = 2, 1, 4, 4
    for a_log, T in ((-3.0, 6), (3.0, 40), (0.5, 300), (-8.0, 300)):
        state = torch.zeros(1, H * N * Pv, device="cuda")
        xbc = torch.randn(T, H * Pv + 2 * G * N, generator=g)
        dt_raw = torch.tensor([[30.0, -30.0], [2.0, 0.0], [-1.0, 8.0]] * ((T + 2) // 3))[:T]
        zeros = torch.zeros(H)
        out = torch.empty(T, H * Pv, device="cuda")
        ops.mamba2_scan(dev(xbc), H * Pv, H * Pv + G * N, dev(dt_raw), dev(zeros), dev(zeros + a_log), dev(zeros), out, state, 0,
                        i32([0, T]), i32([0]), 1, H, G, N, Pv, T, None)
        seg = xbc.to(P.DT)
        y, S = plain_scan(seg[:, :H * Pv].reshape(T, H, Pv), seg[:, H * Pv:H * Pv + N].reshape(T, G, N), seg[:, H * Pv + N:].reshape(T, G, N),
                          dt_raw.to(P.DT), zeros.to(P.DT), zeros.to(P.DT) + a_log, zeros.to(P.DT), torch.zeros(H, N, Pv, dtype=P.DT))
        assert rel_err(out.cpu(), y.reshape(T, H * Pv)) < 2e-5, a_log
        assert rel_err(state.cpu().view(H, N, Pv), S) < 2e-5, a_log


@gpu
def test_the_gate_comes_before_the_norm_and_pieces_are_normed_apart():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    for N, parts, lead in ((48, 2, 2), (30, 3, 2), (64, 1, 2), (4096, 2, 2), (48, 2, 4), (4096, 1, 8), (120, 5, 0)):
        T = 5         # lead 2: the gate's rows start off a 16-byte boundary (scalar kernel); else whole vectors
        y, gate, w = torch.randn(T, N, generator=g) * 2, torch.randn(T, N + 8, generator=g), torch.randn(N, generator=g)
        gated = y.to(P.DT) * P.silu(gate[:, lead:lead + N].to(P.DT))
        want = P.rms_unit(gated.reshape(T, parts, N // parts), 1e-5).reshape(T, N) * w.to(P.DT)
        gd = dev(gate)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            out = torch.empty(T, N, dtype=dtype, device="cuda")
            ops.gated_group_rmsnorm(dev(y), gd[:, lead:lead + N], dev(w), 1e-5, parts, out)
            assert rel_err(out.float().cpu(), want) < tol
        if parts > 1:       # one norm over the whole row is another result
            assert rel_err(P.rms_unit(gated, 1e-5) * w.to(P.DT), want) > 1e-2


# ------------------------------------------------------------------------------------------------
# on the device: each mixer alone in a one-layer model, then whole models
# ------------------------------------------------------------------------------------------------
ALONE = {
    "attention": config(90, 48, 1e-5, 2.0, 0.7, [layer("attention", attention(6, 3, 8, 0.4, mask=70, rot=(6, 500.0, (3.0, 1.0, 2.0, 40))))]),
    "latent": config(90, 48, 1e-5, 2.0, 1.3, [layer("latent_attention", latent(3, 8, 16, 24, 0.4))]),
    "mamba2": config(90, 48, 1e-5, 2.0, 0.9, [layer("mamba2", mamba(4, 12, 10, 2, 3, 4))]),
    "feed_forward": config(90, 48, 1e-5, 2.0, 0.5, [layer("latent_attention", latent(1, 8, 8, 8, 1.0), 100)]),
}


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mixer_alone(tmp_path, name, dtype):
    from janus_b200.engine import StepEntry
    cfg = ALONE[name]
    d, w = folder(tmp_path, cfg, 8)
    model = load(d, dtype)
    seqs = [random_tokens(n, cfg["vocab"], 50 + n) for n in (300, 3, 65)]
    slots = [model.alloc_slot() for _ in seqs]
    out = model.step([StepEntry(s, ids, range(len(ids))) for s, ids in zip(slots, seqs)]).cpu()
    ref = torch.cat([P.forward(cfg, w, ids) for ids in seqs])
    rows = Rows(dtype)
    rows.add(out, ref)
    rows.close()
    model.check()


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
    rows = Rows(dtype)
    at = 0
    for ids in seqs:          # every sequence by itself, the single token too
        rows.add(out[at:at + len(ids)], P.forward(cfg, w, ids), (name, len(ids)))
        at += len(ids)
    rows.close()
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_then_single_tokens_in_a_batch_and_slots_used_again(tmp_path, name, dtype):
    """Prompts cut into portions of 1 to 62 tokens, unequal requests in one batch, then one token each until the
    shorter ones have ended; afterwards other requests take the freed slots, pages and states.  Every row is
    compared with the whole sequence's logits from the plain implementation."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 12)
    rows = Rows(dtype)
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
                rows.add(out[row:row + n], ref[i][lo:lo + n], (round_no, i, lo, n))
                row += n
        live = [0, 1, 2]
        while live:
            out = model.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in live]).cpu()
            for row, i in enumerate(live):
                rows.add(out[row:row + 1], ref[i][at[i]:at[i] + 1], (round_no, i, at[i]))
                at[i] += 1
            for i in [i for i in live if at[i] == len(seqs[i])]:
                model.free_slot(slots[i])
                live.remove(i)
        model.engine.cache.check()
    rows.close()
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_just_inside_and_just_outside_the_window(tmp_path, dtype):
    """One attention layer with peaked attention and one loud token: the plain implementation with the window off
    by one differs clearly from the right one at the rows compared, in prompts, in portions and in single tokens,
    so a key that is seen or missed by mistake would show.  The window passes page borders meanwhile."""
    from janus_b200.engine import StepEntry
    cfg = config(120, 64, 1e-5, 0.1, 1.5, [layer("attention", attention(2, 1, 16, 0.5, mask=70, rot=(8, 10000.0)))])
    w = sharpened(P.random_weights(cfg, 5), 2.0)
    # a loud token: its key points along the dimensions that are not rotated, every query has a large part along
    # them, and its value (the key as projected) is large; only one of them lies in any window
    w["embed"][111] = 0.0
    w["embed"][111, 7] = 8.0
    w["l0.mix.k"][:, 7] = 0.0
    w["l0.mix.k"][8:, 7] = 1.0
    for h in range(2):
        w["l0.mix.q.b"][h * 16 + 8:(h + 1) * 16] = 3.0
    ids = random_tokens(230, cfg["vocab"] - 10, 9)
    for p in (20, 100):
        ids[p] = 111
    d = P.save_folder(cfg, w, str(tmp_path / "edge"))
    ref = P.forward(cfg, w, ids)
    rows = [p + 69 for p in (20, 100)] + [p + 70 for p in (20, 100)]     # the last row that sees it, the first that does not
    for delta in (-1, 1):
        off = copy.deepcopy(cfg)
        off["layers"][0]["mixer"]["mask"]["size"] += delta
        assert rel_err(P.forward(off, w, ids)[rows], ref[rows]) > 0.4, delta
    model = load(d, dtype, max_tokens=512)
    s = model.alloc_slot()
    out = [model.step([StepEntry(s, ids[:88], range(88))]).cpu()]                 # a prompt ...
    out.append(model.step([StepEntry(s, ids[88:92], range(4))]).cpu())            # ... portions over the first edge ...
    out.append(model.step([StepEntry(s, ids[92:160], range(68))]).cpu())
    for t in range(160, 230):                                                     # ... and single tokens
        out.append(model.step([StepEntry(s, [ids[t]], [0])]).cpu())
    out = torch.cat(out)
    assert rel_err(out[rows], ref[rows]) < tol_for(dtype)
    every = Rows(dtype)
    every.add(out, ref)
    every.close()
    held = model.engine.cache.groups[0].pages[s]
    assert held[0] == -1 and held[1] == -1 and held[3] >= 0             # passed pages are given back
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_through_the_latents_and_a_far_token_through_the_state(tmp_path, dtype):
    """Latent attention sees every earlier token: one loud token hundreds of positions back (beyond several pages)
    decides the last logits.  The state-space layer carries a token just as far through its state when a head
    hardly decays.  Changing that one token changes the plain implementation's last logits clearly, and the
    library follows both versions, in a prompt and in single tokens."""
    from janus_b200.engine import StepEntry
    cfg_l = config(90, 32, 1e-5, 0.1, 1.0, [layer("latent_attention", latent(2, 8, 8, 16, 0.5))])
    cfg_m = config(90, 32, 1e-5, 0.1, 1.0, [layer("mamba2", mamba(2, 8, 8, 1, 2, 1))])
    for cfg in (cfg_l, cfg_m):
        w = P.random_weights(cfg, 6)
        for tok, feature in ((5, 0), (77, 1), (12, 2)):
            w["embed"][tok] = 0.0
            w["embed"][tok, feature] = 4.0
        if cfg is cfg_m:
            w["l0.mix.A_log"][:] = -9.0              # next to no decay
            w["l0.mix.dt_bias"][:] = 1.0
            w["l0.mix.in"][16:32, 0] = 0.0           # token 5 writes nothing into the state ...
            w["l0.mix.conv.b"][:16] = 0.0
            w["l0.mix.in"][16:32, 1:3] *= 8.0        # ... the far token writes clearly
        else:
            # the latents of the three tokens are three axes; every head's keys read them off, and the queries of
            # token 5 point away from its own latent and towards the other two
            w["l0.mix.dkv"][:, :3] = 0.0
            w["l0.mix.uk"][:] = 0.0
            w["l0.mix.q"][:, 0] = 0.0
            for f in range(3):
                w["l0.mix.dkv"][f, f] = 1.0
            for h in range(2):
                for f in range(3):
                    w["l0.mix.uk"][h * 8 + f, f] = 1.0
                w["l0.mix.q"][h * 8: h * 8 + 3, 0] = torch.tensor([-8.0, 8.0, 8.0], dtype=P.DT)
        d = P.save_folder(cfg, w, str(tmp_path / ("far" + cfg["layers"][0]["type"])))
        ids = [5] * 400
        ids[3] = 77
        other = list(ids)
        other[3] = 12
        ref, ref_other = P.forward(cfg, w, ids), P.forward(cfg, w, other)
        assert rel_err(ref_other[-5:], ref[-5:]) > 0.4, cfg["layers"][0]["type"]
        model = load(d, dtype, max_tokens=1024)
        for seq, want in ((ids, ref), (other, ref_other)):
            s = model.alloc_slot()
            out = model.step([StepEntry(s, seq[:395], [394])]).cpu()
            assert rel_err(out, want[394:395]) < tol_for(dtype)
            for t in range(395, 400):
                out = model.step([StepEntry(s, [seq[t]], [0])]).cpu()
                assert rel_err(out, want[t:t + 1]) < tol_for(dtype)
            model.free_slot(s)
        model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(tmp_path, dtype):
    """A sequence that starts with a single token and grows by one for 200 steps (replayed CUDA graphs): the
    first tokens (fewer than the convolution's taps, fewer than the window), page borders at 64 and 128, a
    window of 65 keys."""
    from janus_b200.engine import StepEntry
    for name in ("B", "C"):
        cfg = CONFIGS[name]
        d, w = folder(tmp_path, cfg, 13)
        ids = random_tokens(200, cfg["vocab"], 21)
        ref = P.forward(cfg, w, ids)
        model = load(d, dtype, max_tokens=256, max_slots=2)
        s = model.alloc_slot()
        got = [model.step([StepEntry(s, [t], [0])]).cpu() for t in ids]
        rows = Rows(dtype)
        rows.add(torch.cat(got), ref)
        rows.close()
        assert rel_err(torch.cat(got[:6]), ref[:6]) < tol_for(dtype)
        assert model.engine.graph_captures >= 1
        model.check()


def random_config(seed):
    """A configuration drawn from a seed: layer order, every size and every constant."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 64, 96, 128, 136])
    layers, owners = [], {}
    for i in range(rng.randint(3, 7)):
        kind = rng.choice(["attention", "latent_attention", "mamba2"])
        ff = rng.choice([None, 24, 72, 130])
        if kind == "attention":
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([8, 12, 16, 24, 40, 64])
            rot = None
            if rng.random() < 0.8:
                dims = rng.choice([d for d in (4, 8, 12, 16, 24, 40, 64) if d <= dim])
                rot = (dims, rng.choice([50.0, 10000.0]))
                if rng.random() < 0.6:
                    rot += ((rng.choice([2.0, 8.0]), 1.0, rng.choice([2.0, 4.0, 8.0]), rng.choice([16, 64, 256])),)
            m = attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.uniform(0.1, 0.4), mask=rng.choice([None, 3, 17, 64, 100, 136]), rot=rot)
        elif kind == "latent_attention":
            rank = rng.choice([8, 16, 20, 48, 64])
            share = [j for j, r in owners.items() if r == rank]
            kv_from = rng.choice(share) if share and rng.random() < 0.6 else None
            if kv_from is None:
                owners[i] = rank
            m = latent(rng.randint(1, 6), rng.choice([4, 8, 24, 32]), rng.choice([4, 16, 40]), rank, rng.uniform(0.1, 0.5), kv_from)
        else:
            groups = rng.choice([1, 2, 3])
            heads = groups * rng.choice([1, 2])
            vdim = rng.choice([4, 8, 16, 32])
            pieces = rng.choice([g for g in (1, 2, 3, 4, 6) if (heads * vdim) % g == 0])
            m = mamba(heads, vdim, rng.choice([4, 8, 16, 48, 64, 72]), groups, rng.randint(1, 4), pieces)
        layers.append(layer(kind, m, ff))
    return config(rng.choice([80, 130, 257]), width, rng.choice([1e-5, 1e-6]), rng.uniform(0.5, 12.0), rng.uniform(0.4, 1.5), layers)


def test_random_configurations_are_read_and_written_back():
    from janus_b200.config import resolve_architecture
    for seed in range(40):
        cfg = random_config(seed)
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        assert json.loads(json.dumps(c.to_dict())) == json.loads(json.dumps(cfg)), seed
        assert {s.name: tuple(s.shape) for s in arch.weight_specs(c)} == {k: tuple(v.shape) for k, v in P.random_weights(cfg, 0).items()}


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_configurations_in_prompts_portions_and_single_tokens(tmp_path, seed, dtype):
    """Layer order, sizes and constants drawn from a seed; two unequal requests in one batch: a prompt each, a
    portion each, then one token each."""
    from janus_b200.engine import StepEntry
    cfg = random_config(seed)
    d, w = folder(tmp_path, cfg, 40 + seed, sharpen=2.0)
    model = load(d, dtype, max_tokens=1024, max_slots=4)
    seqs = [random_tokens(n, cfg["vocab"], seed * 10 + n) for n in (201, 90)]
    ref = [P.forward(cfg, w, ids) for ids in seqs]
    slots = [model.alloc_slot() for _ in seqs]
    rows = Rows(dtype)
    at = [0, 0]
    for portion in ((150, 3), (40, 64), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1)):
        out = model.step([StepEntry(slots[i], seqs[i][at[i]:at[i] + n], range(n)) for i, n in enumerate(portion)]).cpu()
        row = 0
        for i, n in enumerate(portion):
            rows.add(out[row:row + n], ref[i][at[i]:at[i] + n], (seed, i, at[i], n))
            row += n
            at[i] += n
    rows.close()
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
    """`python -m janus_b200 DIR ...`: greedy tokens equal the plain implementation's picks, and sampling with a
    temperature, top-k and a seed runs through the device sampler; a folder with config.json alone runs with
    `--random-weights`."""
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
