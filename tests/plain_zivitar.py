"""A plain, slow implementation of the Zivitar decoder on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the library.  Everything runs in one
dtype (float64 by default) on whole sequences; `decode_*` variants step token by token with an
explicit state, so that the tests can compare the two ways against each other as well.

Notation: T tokens, W width, H query heads, G key/value heads, d query/key size, e value size,
S residual streams.  Linear weights are [out, in] and applied as W x.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

DT = torch.float64


# ---------------------------------------------------------------------------------------------
# reading a model folder (an independent reader of the file format)
# ---------------------------------------------------------------------------------------------
def read_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        buf = bytearray(data[a:b])
        kind = meta["dtype"]
        if kind == "BF16":
            t = torch.frombuffer(buf, dtype=torch.bfloat16)
        elif kind == "F32":
            t = torch.frombuffer(buf, dtype=torch.float32)
        elif kind == "F16":
            t = torch.frombuffer(buf, dtype=torch.float16)
        elif kind == "I32":
            t = torch.frombuffer(buf, dtype=torch.int32)
        else:
            raise ValueError(f"{name}: stored dtype {kind}")
        t = t.reshape(meta["shape"]).clone()
        out[name] = t.to(DT) if t.is_floating_point() else t
    return cfg, out


# ---------------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def feed_forward(h: torch.Tensor, w_gate, w_up, w_down, limit: float) -> torch.Tensor:
    """g = min(Wg h, limit); u = clamp(Wu h, -limit, limit); Wd (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


# ---------------------------------------------------------------------------------------------
# rotary positions with the ramped frequency scaling
# ---------------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency per pair [dims/2], factor on cos and sin)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    fast, slow = float(scaling["fast"]), float(scaling["slow"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=DT)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, n, d]: the first rot.dims dimensions of each of the n vectors are rotated in the
    pairing (i, i + dims/2); the rest pass."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f, m = rotary_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    a = positions.to(DT)[:, None] * f[None, :]
    c, s = (torch.cos(a) * m)[:, None, :], (torch.sin(a) * m)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------
# the short causal convolution
# ---------------------------------------------------------------------------------------------
def short_conv(u: torch.Tensor, w: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j); `before` [taps - 1, C] holds
    the values just before u (zeros at a sequence's start)."""
    taps = w.shape[1]
    pad = torch.zeros(taps - 1, u.shape[1], dtype=u.dtype) if before is None else before
    full = torch.cat([pad, u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + full[j:j + u.shape[0]] * w[:, j][None, :]
    return y


# ---------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------
def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    if j > i:
        return False
    if not mask:
        return True
    return i - j < int(mask["size"]) or j < int(mask.get("keep_first", 0))


def differential_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                           start: int = 0, state: Optional[dict] = None) -> torch.Tensor:
    """h [T, W] at positions start .. start + T - 1.  `state` (for stepping) carries the projected
    values before the convolution and the keys and values of earlier positions."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if m.get("conv"):
        taps = int(m["conv"])
        prev = state.get("conv") if state is not None else None
        if state is not None:
            allp = torch.cat([q, k, v], dim=1)
            joined = allp if prev is None else torch.cat([prev, allp], dim=0)
            if joined.shape[0] < taps - 1:
                joined = torch.cat([torch.zeros(taps - 1 - joined.shape[0], joined.shape[1], dtype=DT), joined])
            state["conv"] = joined[joined.shape[0] - (taps - 1):]
        nq, nk = q.shape[1], k.shape[1]
        pq = pk = pv = None
        if prev is not None:
            pq, pk, pv = prev[:, :nq], prev[:, nq:nq + nk], prev[:, nq + nk:]
        q, k, v = short_conv(q, w["q.conv"], pq), short_conv(k, w["k.conv"], pk), short_conv(v, w["v.conv"], pv)
    pos = torch.arange(start, start + T)
    q = rotate(q.view(T, H * 2, d), pos, m.get("rot")).view(T, H, 2, d)
    k = rotate(k.view(T, G * 2, d), pos, m.get("rot")).view(T, G, 2, d)
    v = v.view(T, G, e)
    if state is not None:
        if "k" in state:
            k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
        state["k"], state["v"] = k, v
    diff = float(m["diff"])
    lam = math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff
    scale = float(m["scale"])
    out = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        i = start + t
        keys = [j for j in range(i + 1) if visible(i, j, m.get("mask"))]
        for hh in range(H):
            g = hh // (H // G)
            maps = []
            for mp in range(2):
                s = (k[keys, g, mp] @ q[t, hh, mp]) * scale
                p = torch.softmax(s, dim=0)
                maps.append(p @ v[keys, g])
            o = maps[0] - lam * maps[1]
            out[t, hh] = rms_unit(o, eps) * (1.0 - diff)
    return out.reshape(T, H * e) @ w["o"].T


def lightning_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                        state: Optional[dict] = None) -> torch.Tensor:
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; heads joined, normed, gated, projected."""
    T = h.shape[0]
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w["q"].T).view(T, H, d)
    k = silu(h @ w["k"].T).view(T, H, d)
    v = silu(h @ w["v"].T).view(T, H, e)
    decay = torch.tensor(m["decay"], dtype=DT)
    S = torch.zeros(H, d, e, dtype=DT) if state is None or "S" not in state else state["S"]
    o = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    if state is not None:
        state["S"] = S
    y = rms_norm(o.reshape(T, H * e), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return y @ w["o"].T


# ---------------------------------------------------------------------------------------------
# the whole model
# ---------------------------------------------------------------------------------------------
def _sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def owner_of(cfg: dict, i: int) -> int:
    while cfg["layers"][i].get("weights_of") is not None:
        i = int(cfg["layers"][i]["weights_of"])
    return i


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], start: int = 0,
            states: Optional[list] = None, layer_sums: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of the tokens `ids` at positions start ..; `states` (one dict per layer
    of the configuration, kept by the caller) lets a sequence be fed in pieces."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(ids)]
    S = cfg.get("streams")
    streams = [x.clone() for _ in range(int(S))] if S else None

    def sublayer(q: int, p: str, fn, norm_w):
        nonlocal x, streams
        if streams is None:
            x = x + fn(rms_norm(x, norm_w, eps))
            return
        c_in, c_out, c_mix = w[p + f"hc{q}.in"], w[p + f"hc{q}.out"], w[p + f"hc{q}.mix"]
        u = sum(c_in[s] * streams[s] for s in range(len(streams)))
        y = fn(rms_norm(u, norm_w, eps))
        streams = [sum(c_mix[s, t] * streams[s] for s in range(len(streams))) + c_out[t] * y
                   for t in range(len(streams))]

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner_of(cfg, i)}."
        mw = _sub(w, p + "mix.")
        st = states[i] if states is not None else None
        if layer["type"] == "lightning":
            mixer = lambda z: lightning_attention(z, mw, layer["mixer"], eps, st)       # noqa: E731
        elif layer["type"] == "attention":
            mixer = lambda z: differential_attention(z, mw, layer["mixer"], eps, start, st)   # noqa: E731
        else:
            raise ValueError(layer["type"])
        sublayer(1, p, mixer, w[p + "norm1"])
        if layer.get("mlp") is not None:
            fw = _sub(w, p + "mlp.")
            sublayer(2, p, lambda z: feed_forward(z, fw["gate"], fw["up"], fw["down"], float(layer["mlp"]["limit"])),
                     w[p + "norm2"])
        if layer_sums is not None:
            layer_sums.append(sum(streams) if streams is not None else x)
    if streams is not None:
        x = sum(streams)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    if cfg.get("logit_scale") is not None:
        logits = logits * float(cfg["logit_scale"])
    if cfg.get("logit_softcap") is not None:
        cap = float(cfg["logit_softcap"])
        logits = cap * torch.tanh(logits / cap)
    return logits


def forward_in_pieces(cfg: dict, w, ids: List[int], cuts: List[int]) -> torch.Tensor:
    """The same logits with the sequence fed piece by piece (`cuts`: piece lengths) through states."""
    states = [dict() for _ in cfg["layers"]]
    out, at = [], 0
    for n in cuts:
        out.append(forward(cfg, w, ids[at:at + n], at, states))
        at += n
    return torch.cat(out)


def random_weights(cfg: dict, seed: int, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Random tensors for a configuration, rounded to bfloat16 values (as a stored model's are)."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])

    def rnd(*shape, s=std, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).to(DT)

    w = {"embed": rnd(cfg["vocab"], W, s=1.0), "final.norm": rnd(W, s=0.1, mean=1.0), "head": rnd(cfg["vocab"], W, s=W ** -0.5)}
    S = cfg.get("streams")
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = rnd(W, s=0.1, mean=1.0)
        if layer["type"] == "lightning":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * e), ("g", H * e)):
                w[p + "mix." + n] = rnd(rows, W, s=W ** -0.5)
            w[p + "mix.o"] = rnd(W, H * e, s=(H * e) ** -0.5)
            w[p + "mix.norm"] = rnd(H * e, s=0.1, mean=1.0)
        else:
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * 2 * d), ("k", G * 2 * d), ("v", G * e)):
                w[p + "mix." + n] = rnd(rows, W, s=W ** -0.5)
                if m.get("conv"):
                    w[p + f"mix.{n}.conv"] = rnd(rows, m["conv"], s=0.5)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[p + "mix." + n] = rnd(d, s=0.1)
            w[p + "mix.o"] = rnd(W, H * e, s=(H * e) ** -0.5)
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            w[p + "norm2"] = rnd(W, s=0.1, mean=1.0)
            w[p + "mlp.gate"], w[p + "mlp.up"] = rnd(F, W, s=W ** -0.5), rnd(F, W, s=W ** -0.5)
            w[p + "mlp.down"] = rnd(W, F, s=F ** -0.5)
        if S:
            for q in ((1, 2) if layer.get("mlp") is not None else (1,)):
                w[p + f"hc{q}.in"] = rnd(S, s=0.2, mean=1.0 / S)
                w[p + f"hc{q}.out"] = rnd(S, s=0.2, mean=1.0)
                w[p + f"hc{q}.mix"] = (torch.eye(S) + torch.randn(S, S, generator=g) * 0.1).to(torch.bfloat16).to(DT)
    return w


def save_folder(cfg: dict, w: Dict[str, torch.Tensor], out_dir: str, dtype=torch.bfloat16) -> str:
    """Write config.json and model.safetensors (an independent writer of the file format)."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    names = {torch.bfloat16: "BF16", torch.float32: "F32"}
    for name, t in w.items():
        t = t.to(dtype).contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(out_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return out_dir


def as_numpy(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float64).numpy()
