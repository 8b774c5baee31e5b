"""A plain, slow implementation of the Ramolix decoder on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the library.  Everything runs in one
dtype (float64) on whole sequences; the mixers take and return an explicit state, so that the
tests can run a sequence in one piece, in portions or token by token and compare.

Notation: T tokens, W width, H query heads, G key/value heads (or groups), d query/key size,
e value size, r latent size, N state size, P value size of a state-space head.
Linear weights are [out, in] and applied as W x.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

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
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[meta["dtype"]]).reshape(meta["shape"]).clone()
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


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def feed_forward(h: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """Wd (gelu_tanh(Wg h) * (Wu h))"""
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


# ---------------------------------------------------------------------------------------------
# rotary positions, frequencies scaled band by band
# ---------------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """One frequency per pair.  With scaling (factor, low, high, original) and wavelength
    l = 2 pi / f: short waves (l < original / high) keep f, long waves (l > original / low) get
    f / factor, the band between is blended linearly in original / l."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            wave = 2.0 * math.pi / f
            if wave > original / low:
                f = f / factor
            elif wave >= original / high:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=DT)


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, n, d]: the first rot.dims dimensions of each vector are turned in the pairing
    (i, i + dims/2); the rest pass."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f = rotary_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    a = positions.to(DT)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------
# softmax attention over explicit keys
# ---------------------------------------------------------------------------------------------
def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor, scale: float, window: int):
    """q [T, H, d] at positions q_pos; k [L, G, d], v [L, G, e] at positions 0..L-1; head h uses key/value
    head floor(h / (H / G)); position i sees j with 0 <= i - j (< window, if window > 0).  Returns [T, H, e]."""
    T, H, _ = q.shape
    L, G, e = v.shape
    out = torch.zeros((T, H, e), dtype=DT)
    j = torch.arange(L)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h, :] @ k[:, g, :].T) * scale                      # [T, L]
        dist = q_pos[:, None] - j[None, :]
        seen = dist >= 0
        if window > 0:
            seen = seen & (dist < window)
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    return out


# ---------------------------------------------------------------------------------------------
# mixer: sliding-window attention whose values are the projected keys
# ---------------------------------------------------------------------------------------------
def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, state: Optional[dict]):
    """state: {"k": rotated keys so far [L, G, d], "v": values so far [L, G, d]} or None at a sequence's start."""
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    T = h.shape[0]
    start = 0 if state is None else state["k"].shape[0]
    pos = torch.arange(start, start + T)
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    v = k.reshape(T, G, d)                                           # the values: the keys as projected
    q = rms_norm(q, w["q.norm"], eps).reshape(T, H, d)               # one root mean square over all heads
    k = rms_norm(k, w["k.norm"], eps).reshape(T, G, d)
    q, k = rotate(q, pos, m.get("rot")), rotate(k, pos, m.get("rot"))
    if state is not None:
        k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    o = attend(q, k, v, pos, float(m["scale"]), window)
    return o.reshape(T, H * d) @ w["o"].T, {"k": k, "v": v}


# ---------------------------------------------------------------------------------------------
# mixer: latent attention (keys and values are made from a small cached vector per token)
# ---------------------------------------------------------------------------------------------
def latent_of(h: torch.Tensor, w: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    return rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, latents: torch.Tensor):
    """latents [L, r]: the latent vectors of the whole sequence up to and including this portion's
    tokens (its own layer's, or the layer's that `kv_from` names)."""
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T, L = h.shape[0], latents.shape[0]
    pos = torch.arange(L - T, L)
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (latents @ w["uk"].T).reshape(L, H, d)
    v = (latents @ w["uv"].T).reshape(L, H, e)
    o = attend(q, k, v, pos, float(m["scale"]), 0)
    return o.reshape(T, H * e) @ w["o"].T


# ---------------------------------------------------------------------------------------------
# mixer: the selective state-space recurrence
# ---------------------------------------------------------------------------------------------
def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, state: Optional[dict]):
    """state: {"conv": the last taps - 1 inputs of the convolution [taps - 1, C], "ssm": [heads, N, P]}."""
    heads, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    taps, parts = int(m["conv"]), int(m["norm_groups"])
    inner, T = heads * P, h.shape[0]
    C = inner + 2 * G * N
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
    before = torch.zeros((taps - 1, C), dtype=DT) if state is None else state["conv"]
    padded = torch.cat([before, xbc])
    conv = torch.zeros((T, C), dtype=DT)
    for j in range(taps):                                            # the last column meets the current token
        conv = conv + padded[j:j + T] * w["conv"][:, j]
    xbc_act = silu(conv + w["conv.b"])
    x = xbc_act[:, :inner].reshape(T, heads, P)
    B = xbc_act[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc_act[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])                                 # [T, heads]
    A = -torch.exp(w["A_log"])
    S = torch.zeros((heads, N, P), dtype=DT) if state is None else state["ssm"].clone()
    y = torch.zeros((T, heads, P), dtype=DT)
    for t in range(T):
        for i in range(heads):
            g = i // (heads // G)
            S[i] = torch.exp(A[i] * dt[t, i]) * S[i] + dt[t, i] * torch.outer(B[t, g], x[t, i])
            y[t, i] = S[i].T @ Cm[t, g] + w["D"][i] * x[t, i]
    y = y.reshape(T, inner) * silu(z)                                # the gate comes before the norm
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T, {"conv": padded[padded.shape[0] - (taps - 1):], "ssm": S}


# ---------------------------------------------------------------------------------------------
# the whole model
# ---------------------------------------------------------------------------------------------
def _sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


class PlainRamolix:
    """Runs sequences in portions of any size; `states[seq]` carries what a sequence has left."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, {k: v.to(DT) for k, v in weights.items()}
        self.eps = float(cfg["norm"]["eps"])
        self.states: Dict[object, List[Optional[dict]]] = {}

    def forget(self, seq) -> None:
        self.states.pop(seq, None)

    def forward(self, seq, tokens, keep_layers: bool = False):
        """The logits [T, vocab] of this portion's tokens (and, if asked for, the residual stream after every layer)."""
        cfg, w, eps = self.cfg, self.w, self.eps
        layers = cfg["layers"]
        st = self.states.setdefault(seq, [None] * len(layers))
        mult = float(cfg["residual_mult"])
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
        after = []
        for i, layer in enumerate(layers):
            p, m = f"l{i}.", layer["mixer"]
            mw = _sub(w, p + "mix.")
            if layer["type"] == "attention":
                y, st[i] = window_attention(x, mw, m, eps, st[i])
            elif layer["type"] == "mamba2":
                y, st[i] = mamba2(x, mw, m, eps, st[i])
            elif layer["type"] == "latent_attention":
                if m.get("kv_from") is None:
                    c = latent_of(x, mw, eps)
                    st[i] = {"c": c if st[i] is None else torch.cat([st[i]["c"], c])}
                    latents = st[i]["c"]
                else:
                    latents = st[int(m["kv_from"])]["c"]
                y = latent_attention(x, mw, m, latents)
            else:
                raise ValueError(layer["type"])
            x = x + mult * rms_norm(y, w[p + "norm1"], eps)
            if layer.get("mlp") is not None:
                fw = _sub(w, p + "mlp.")
                x = x + mult * rms_norm(feed_forward(x, fw["gate"], fw["up"], fw["down"]), w[p + "norm2"], eps)
            if keep_layers:
                after.append(x.clone())
        logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
        return (logits, torch.stack(after)) if keep_layers else logits


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int]) -> torch.Tensor:
    """The logits [T, vocab] of a whole sequence."""
    return PlainRamolix(cfg, w).forward(0, ids)


def forward_in_pieces(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], cuts: List[int]) -> torch.Tensor:
    """The same logits with the sequence fed piece by piece (`cuts`: piece lengths) through the states."""
    m = PlainRamolix(cfg, w)
    out, at = [], 0
    for n in cuts:
        out.append(m.forward(0, ids[at:at + n]))
        at += n
    return torch.cat(out)


# ---------------------------------------------------------------------------------------------
# random models
# ---------------------------------------------------------------------------------------------
def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random tensors for a configuration, rounded to bfloat16 values (as a stored model's are)."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).to(DT)

    w = {"embed": rnd(cfg["vocab"], W), "final.norm": rnd(W, s=0.1, mean=1.0)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = rnd(W, s=0.1, mean=1.0)
        if layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            w[p + "mix.q"], w[p + "mix.k"] = rnd(H * d, W, s=W ** -0.5), rnd(G * d, W, s=W ** -0.5)
            w[p + "mix.q.b"], w[p + "mix.k.b"] = rnd(H * d, s=0.2), rnd(G * d, s=0.2)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = rnd(H * d, s=0.2, mean=1.0), rnd(G * d, s=0.2, mean=1.0)
            w[p + "mix.o"] = rnd(W, H * d, s=(H * d) ** -0.5)
        elif layer["type"] == "latent_attention":
            H, d, e, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"] = rnd(H * d, W, s=W ** -0.5)
            if m.get("kv_from") is None:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = rnd(r, W, s=W ** -0.5), rnd(r, s=0.2, mean=1.0)
            w[p + "mix.uk"], w[p + "mix.uv"] = rnd(H * d, r, s=r ** -0.5), rnd(H * e, r, s=r ** -0.5)
            w[p + "mix.o"] = rnd(W, H * e, s=(H * e) ** -0.5)
        else:
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * P, H * P + 2 * G * N
            w[p + "mix.in"] = rnd(2 * inner + 2 * G * N + H, W, s=W ** -0.5)
            w[p + "mix.conv"], w[p + "mix.conv.b"] = rnd(C, taps, s=taps ** -0.5), rnd(C, s=0.2)
            w[p + "mix.dt_bias"], w[p + "mix.A_log"] = rnd(H, s=0.7), rnd(H, s=0.7, mean=-1.0)
            w[p + "mix.D"], w[p + "mix.norm"] = rnd(H, s=0.3, mean=1.0), rnd(inner, s=0.1, mean=1.0)
            w[p + "mix.o"] = rnd(W, inner, s=inner ** -0.5)
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            w[p + "norm2"] = rnd(W, s=0.1, mean=1.0)
            w[p + "mlp.gate"], w[p + "mlp.up"] = rnd(F, W, s=W ** -0.5), rnd(F, W, s=W ** -0.5)
            w[p + "mlp.down"] = rnd(W, F, s=F ** -0.5)
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
