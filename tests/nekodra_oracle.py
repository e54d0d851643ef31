"""Plain, slow fp32 statement of the Nekodra decoder, one function per mechanism (torch on the CPU).

Shares no code with the product path: the tests build small random models, run them through the
library and compare with these functions. Shapes: T tokens, D model width, H heads, dq query/key
size per head, dv value size per head, R latent size, E routed experts, I identity experts.

A model is (config dict as in config.json, dict name -> torch.float32 tensor).
"""
import math

import torch


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations"""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def latent(h, w_dkv, w_norm, eps):
    """the cached row of a token: RMS-normed down projection, [T, R]"""
    return rms_norm(h @ w_dkv.T, w_norm, eps)


def sink_attention(q, k, v, scale, sink):
    """Causal attention of ONE head whose softmax denominator also holds exp(sink) (no key, no value).

    q [T, dq] are the LAST T positions of a sequence with keys k [S, dq], values v [S, dv], S >= T.
    """
    T, S = q.shape[0], k.shape[0]
    s = (q @ k.T) * scale                                   # [T, S]
    pos_q = torch.arange(S - T, S).unsqueeze(1)
    pos_k = torch.arange(S).unsqueeze(0)
    s = s.masked_fill(pos_k > pos_q, float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.reshape(1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True) + torch.exp(sink - m)
    return (e / den) @ v


def latent_attention(h, c_all, p, mx, eps):
    """Mixer output for the last T tokens. h [T, D] mixer input; c_all [S, R] the latents of the whole sequence
    (own layer's or the layer named by kv_from); p: dict of this layer's mixer tensors (q, uk, uv, sink, g, o)."""
    H, dq, dv = mx["heads"], mx["dim"], mx["vdim"]
    q = h @ p["q"].T                                        # [T, H*dq]
    k = c_all @ p["uk"].T                                   # [S, H*dq]
    v = c_all @ p["uv"].T                                   # [S, H*dv]
    heads = []
    for i in range(H):
        heads.append(sink_attention(q[:, i * dq:(i + 1) * dq], k[:, i * dq:(i + 1) * dq], v[:, i * dv:(i + 1) * dv],
                                    mx["scale"], p["sink"][i]))
    a = torch.cat(heads, -1) * torch.sigmoid(h @ p["g"].T)
    return a @ p["o"].T


def glu_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, w_router, correction, top, scale):
    """-> (chosen [T, top] expert ids, weights [T, top]). Softmax over ALL router outputs; the choice uses the
    corrected scores, the weights the uncorrected ones times scale, not renormalised."""
    s = torch.softmax(h @ w_router.T, -1)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * scale


def moe(h, p, ml):
    """p: dict with router, correction, e<i>.{gate,up,down}, shared.{gate,up,down}; ml the layer's 'mlp' config.
    The last `identity` router outputs are identity experts (output = input)."""
    r = ml["router"]
    E = r["experts"]
    chosen, w = route(h, p["router"], p["correction"], r["top"], r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(chosen[t, j])
            if e >= E:
                out[t] += w[t, j] * h[t]
            else:
                out[t] += w[t, j] * glu_expert(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if ml.get("shared"):
        out = out + glu_expert(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


class Oracle:
    """Whole-sequence forward with a list of per-layer latents (recomputed from scratch on every call)."""

    def __init__(self, config, weights):
        self.cfg, self.w = config, {k: v.float() for k, v in weights.items()}

    def forward(self, tokens, return_layers=False):
        """logits [T, vocab] of a whole sequence from position 0 (and the residual after every layer)"""
        cfg, w = self.cfg, self.w
        eps = cfg["norm"]["eps"]
        ids = torch.as_tensor(tokens, dtype=torch.long)
        x = w["embed"][ids] + w["pos"][: len(ids)]
        lat, trail = {}, []
        for i, layer in enumerate(cfg["layers"]):
            assert layer["type"] == "latent_attention"
            pre = f"l{i}."
            h1 = layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps)
            h2 = layer_norm(x, w[pre + "norm2"], w[pre + "norm2.b"], eps)
            mx, p = layer["mixer"], sub(w, pre + "mix.")
            if "kv_from" in mx:
                c = lat[mx["kv_from"]]
            else:
                c = lat[i] = latent(h1, p["dkv"], p["dkv.norm"], eps)
            y = latent_attention(h1, c, p, mx, eps)
            if layer.get("mlp"):
                y = y + moe(h2, sub(w, pre + "mlp."), layer["mlp"])
            x = x + y
            trail.append(x)
        logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
        return (logits, torch.stack(trail)) if return_layers else logits

    def greedy(self, prompt, n_new):
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(self.forward(ids)[-1].argmax()))
        return ids[len(prompt):]


def random_model(seed, width=64, vocab=97, max_positions=256, layers=None, eps=1e-5, std=None):
    """A small random model of the design. `layers`: list of dicts with heads, dim, vdim, kv_rank, scale, optional
    kv_from, and an 'mlp' dict (or None). Returns (config, weights as float32 tensors rounded to bfloat16 values)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        s = s if s is not None else (std if std is not None else 1.0 / math.sqrt(shape[-1]))
        return (torch.randn(*shape, generator=g) * s).bfloat16().float()

    if layers is None:
        mlp = dict(kind="moe", expert=dict(ff=48), router=dict(experts=5, identity=2, top=3, scale=1.25), shared=dict(ff=32))
        layers = [dict(heads=3, dim=16, vdim=24, kv_rank=40, scale=0.25, mlp=mlp),
                  dict(heads=3, dim=16, vdim=24, kv_rank=40, scale=0.25, kv_from=0, mlp=mlp)]
    cfg = dict(architecture="Nekodra", vocab=vocab, width=width, max_positions=max_positions, norm=dict(eps=eps), layers=[])
    w = {"embed": rnd(vocab, width, s=1.0), "pos": rnd(max_positions, width, s=0.5)}
    for i, L in enumerate(layers):
        H, dq, dv, R = L["heads"], L["dim"], L["vdim"], L["kv_rank"]
        mx = dict(heads=H, dim=dq, vdim=dv, kv_rank=R, scale=L["scale"])
        pre = f"l{i}."
        for n in ("norm1", "norm2"):
            w[pre + n] = (1 + 0.2 * torch.randn(width, generator=g)).bfloat16().float()
            w[pre + n + ".b"] = rnd(width, s=0.1)
        w[pre + "mix.q"] = rnd(H * dq, width)
        if "kv_from" in L:
            mx["kv_from"] = L["kv_from"]
        else:
            w[pre + "mix.dkv"] = rnd(R, width)
            w[pre + "mix.dkv.norm"] = (1 + 0.2 * torch.randn(R, generator=g)).bfloat16().float()
        w[pre + "mix.uk"] = rnd(H * dq, R, s=2.0 / math.sqrt(R))
        w[pre + "mix.uv"] = rnd(H * dv, R)
        w[pre + "mix.sink"] = rnd(H, s=1.0)
        w[pre + "mix.g"] = rnd(H * dv, width)
        w[pre + "mix.o"] = rnd(width, H * dv)
        ml = L.get("mlp")
        if ml:
            r = ml["router"]
            for e in range(r["experts"]):
                w[pre + f"mlp.e{e}.gate"] = rnd(ml["expert"]["ff"], width)
                w[pre + f"mlp.e{e}.up"] = rnd(ml["expert"]["ff"], width)
                w[pre + f"mlp.e{e}.down"] = rnd(width, ml["expert"]["ff"])
            n_out = r["experts"] + r["identity"]
            w[pre + "mlp.router"] = rnd(n_out, width, s=2.0 / math.sqrt(width))
            w[pre + "mlp.correction"] = rnd(n_out, s=0.05)
            if ml.get("shared"):
                f = ml["shared"]["ff"]
                w[pre + "mlp.shared.gate"] = rnd(f, width)
                w[pre + "mlp.shared.up"] = rnd(f, width)
                w[pre + "mlp.shared.down"] = rnd(width, f)
        cfg["layers"].append(dict(type="latent_attention", mixer=mx, mlp=ml))
    w["final.norm"] = (1 + 0.2 * torch.randn(width, generator=g)).bfloat16().float()
    w["final.norm.b"] = rnd(width, s=0.1)
    w["head"] = rnd(vocab, width)
    return cfg, w


def write_model(folder, cfg, weights):
    """config.json + model.safetensors (bfloat16; int tensors as int32) in `folder`"""
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
