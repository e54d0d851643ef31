"""Plain, slow statement of the Musilorn decoder, one function per mechanism (torch on the CPU, float64 by default).

Shares no code with the product path: the tests build small random models, run them through the library and
compare with these functions. Every function sees a WHOLE sequence from position 0; nothing is cached.

Design: sandwich layers x <- x + m * LN_b(sub(LN_a(x))) for a mixer and (optionally) a dense GLU feed-forward with
tanh-gelu; two mixers: "attention" (grouped query heads, a short causal convolution over time on the projected q and k,
per-head RMS norm with a shared weight, interleaved rotary positions with long-context frequency scaling, values =
the convolved keys, tanh-capped scores, one added to the softmax denominator) and "retention" (per-head fixed decay,
rotate-half rotary positions, a state S <- decay * S + k v^T, unit-RMS outputs, a silu gate). A span of layers is run
several times with the same weights; each pass starts with a projection of [x; embedding].

A model is (config dict as in config.json, dict name -> tensor).
"""
import math

import torch

DT = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rot_frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2; with rot['scaling']: wavelengths above original/low are stretched by factor,
    those below original/high are kept, the band between is blended linearly in original/wavelength."""
    n = rot["dims"] // 2
    f = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(n)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wl = 2 * math.pi / fi
            if wl < sc["original"] / sc["high"]:
                out.append(fi)
            elif wl > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=DT)


def rotate(x, rot, layout, first_pos=0):
    """x [T, heads, dim]; rotates the first rot['dims'] dimensions of every head. layout 'half': dimension i pairs with
    i + dims/2; 'interleaved': 2i pairs with 2i + 1."""
    T, d = x.shape[0], rot["dims"]
    ang = torch.arange(first_pos, first_pos + T, dtype=DT)[:, None] * rot_frequencies(rot)[None, :]   # [T, d/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., : d // 2], x[..., d // 2: d]
        out[..., : d // 2] = u * c - v * s
        out[..., d // 2: d] = v * c + u * s
    else:
        u, v = x[..., 0:d:2], x[..., 1:d:2]
        out[..., 0:d:2] = u * c - v * s
        out[..., 1:d:2] = v * c + u * s
    return out


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start"""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def capped_sink_attention(q, k, v, scale, cap):
    """ONE head, whole sequence. scores (q.k) * scale, then cap * tanh(score / cap), causal,
    p_j = exp(s_j) / (1 + sum exp(s_j))."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for i in range(T):
        s = (k[: i + 1] @ q[i]) * scale
        s = cap * torch.tanh(s / cap)
        m = max(float(s.max()), 0.0)
        e = torch.exp(s - m)
        out[i] = (e / (e.sum() + math.exp(-m))) @ v[: i + 1]
    return out


def attention_mixer(h, p, mx, eps):
    """h [T, D]; p: this layer's mixer tensors (q, k, q.conv, k.conv, q.norm, k.norm, o)"""
    T, H, G, dim = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"]
    assert mx["vdim"] == dim        # the values are the keys
    q = short_conv(h @ p["q"].T, p["q.conv"]).reshape(T, H, dim)
    k = short_conv(h @ p["k"].T, p["k.conv"]).reshape(T, G, dim)
    v = k
    q = rotate(unit_rms(q, eps) * p["q.norm"], mx["rot"], "interleaved")
    k = rotate(unit_rms(k, eps) * p["k.norm"], mx["rot"], "interleaved")
    heads = [capped_sink_attention(q[:, i], k[:, i // (H // G)], v[:, i // (H // G)], mx["scale"], mx["softcap"]) for i in range(H)]
    return torch.cat(heads, -1) @ p["o"].T


def retention_state_walk(q, k, v, decay):
    """ONE head: S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, S before the first token = 0"""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=q.dtype)
    out = []
    for t in range(q.shape[0]):
        S = decay * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def retention_mixer(h, p, mx, eps):
    """p: q, k, v, g, o"""
    T, H, dim, vdim = h.shape[0], mx["heads"], mx["dim"], mx["vdim"]
    q = rotate((h @ p["q"].T).reshape(T, H, dim), mx["rot"], "half")
    k = rotate((h @ p["k"].T).reshape(T, H, dim), mx["rot"], "half") * dim ** -0.5
    v = (h @ p["v"].T).reshape(T, H, vdim)
    o = torch.stack([retention_state_walk(q[:, i], k[:, i], v[:, i], mx["decay"][i]) for i in range(H)], 1)   # [T, H, vdim]
    o = unit_rms(o, eps).reshape(T, H * vdim)
    return (o * silu(h @ p["g"].T)) @ p["o"].T


def dense_ff(h, p):
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def capped(z, cap):
    return cap * torch.tanh(z / cap)


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_runs(cfg):
    """[(layer index, first of a pass?)] in the order they run"""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    span = list(range(lp["start"], lp["stop"]))
    order = [(i, False) for i in range(lp["start"])]
    for _ in range(lp["times"]):
        order += [(i, i == lp["start"]) for i in span]
    return order + [(i, False) for i in range(lp["stop"], n)]


class Oracle:
    def __init__(self, config, weights, dtype=DT):
        self.cfg, self.w = config, {k: v.to(dtype) for k, v in weights.items()}

    def forward(self, tokens, return_layers=False):
        """logits [T, vocab] of a whole sequence from position 0 (and the residual after every layer run)"""
        cfg, w = self.cfg, self.w
        eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
        x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        x, trail = x0, []
        for i, pass_start in layer_runs(cfg):
            layer, pre = cfg["layers"][i], f"l{i}."
            if pass_start:
                x = torch.cat([x, x0], -1) @ w["loop.in"].T
            mixer = {"attention": attention_mixer, "retention": retention_mixer}[layer["type"]]
            y = mixer(layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps), sub(w, pre + "mix."), layer["mixer"], eps)
            x = x + m * layer_norm(y, w[pre + "norm1b"], w[pre + "norm1b.b"], eps)
            if layer.get("mlp"):
                assert layer["mlp"]["kind"] == "dense"
                y = dense_ff(layer_norm(x, w[pre + "norm2"], w[pre + "norm2.b"], eps), sub(w, pre + "mlp."))
                x = x + m * layer_norm(y, w[pre + "norm2b"], w[pre + "norm2b.b"], eps)
            trail.append(x)
        logits = capped(layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T, cfg["logit_softcap"])
        return (logits, torch.stack(trail)) if return_layers else logits

    def greedy(self, prompt, n_new):
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(self.forward(ids)[-1].argmax()))
        return ids[len(prompt):]


def random_model(seed, width=48, vocab=61, layers=None, loop=None, eps=1e-5, residual_mult=0.4, logit_softcap=12.0):
    """A small random model of the design. `layers`: list of dicts, each with type ('attention' / 'retention'), the mixer's
    sizes and 'ff' (or None for a layer without feed-forward). Returns (config, weights rounded to bfloat16 values)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        s = s if s is not None else 1.0 / math.sqrt(shape[-1])
        return (torch.randn(*shape, generator=g) * s).bfloat16().float()

    def norm(prefix, n):
        w[prefix] = (1 + 0.2 * torch.randn(n, generator=g)).bfloat16().float()
        w[prefix + ".b"] = rnd(n, s=0.1)

    cfg = dict(architecture="Musilorn", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=residual_mult,
               logit_softcap=logit_softcap, layers=[])
    w = {"embed": rnd(vocab, width, s=1.0)}
    if loop:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
        w["loop.in"] = rnd(width, 2 * width, s=1.0 / math.sqrt(width))
    for i, L in enumerate(layers):
        pre = f"l{i}."
        norm(pre + "norm1", width)
        norm(pre + "norm1b", width)
        H, dim = L["heads"], L["dim"]
        if L["type"] == "attention":
            G, taps = L.get("kv_heads", H), L.get("conv", 4)
            mx = dict(heads=H, kv_heads=G, dim=dim, vdim=dim, conv=taps, scale=L.get("scale", dim ** -0.5), softcap=L.get("softcap", 20.0),
                      rot=dict(base=L.get("base", 10000.0), dims=L.get("rot_dims", dim)))
            if L.get("scaling"):
                mx["rot"]["scaling"] = L["scaling"]
            w[pre + "mix.q"], w[pre + "mix.k"] = rnd(H * dim, width, s=2.0 / math.sqrt(width)), rnd(G * dim, width, s=2.0 / math.sqrt(width))
            w[pre + "mix.q.conv"], w[pre + "mix.k.conv"] = rnd(H * dim, taps, s=0.6), rnd(G * dim, taps, s=0.6)
            w[pre + "mix.q.norm"] = (1 + 0.3 * torch.randn(dim, generator=g)).bfloat16().float()
            w[pre + "mix.k.norm"] = (1 + 0.3 * torch.randn(dim, generator=g)).bfloat16().float()
            w[pre + "mix.o"] = rnd(width, H * dim)
        else:
            vdim = L["vdim"]
            mx = dict(heads=H, dim=dim, vdim=vdim, decay=L["decay"], rot=dict(base=L.get("base", 10000.0), dims=L.get("rot_dims", dim)))
            w[pre + "mix.q"], w[pre + "mix.k"] = rnd(H * dim, width), rnd(H * dim, width)
            w[pre + "mix.v"], w[pre + "mix.g"] = rnd(H * vdim, width), rnd(H * vdim, width)
            w[pre + "mix.o"] = rnd(width, H * vdim)
        ml = None
        if L.get("ff"):
            ml = dict(kind="dense", ff=L["ff"])
            norm(pre + "norm2", width)
            norm(pre + "norm2b", width)
            w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"] = rnd(L["ff"], width), rnd(L["ff"], width), rnd(width, L["ff"])
        cfg["layers"].append(dict(type=L["type"], mixer=mx, mlp=ml))
    norm("final.norm", width)
    w["head"] = rnd(vocab, width)
    return cfg, w


def write_model(folder, cfg, weights):
    """config.json + model.safetensors (bfloat16) in `folder`"""
    import json
    import os
    import struct

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        raw = t.bfloat16().contiguous().view(torch.int16).numpy().tobytes()
        header[name] = dict(dtype="BF16", shape=list(t.shape), data_offsets=[off, off + len(raw)])
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
