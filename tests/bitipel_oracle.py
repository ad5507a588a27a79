"""Plain, slow restatement of the Bitipel decoder in float64 torch on the CPU: one function per mechanism, written from
the equations alone.  It shares no code with the package: tests compare the framework's kernels, cache and scheduler
against it.  Weights are a dict {tensor name: tensor} with the checkpoint's names, the configuration is the dict that
config.json holds.

Notation: W = width, H = heads, dn / dr = unrotated / rotated query-key size per head, dv = value size per head,
R = latent size, E = experts, m = residual multiplier.  A linear weight is stored [out][in]: y = M @ x.
"""
import math

import torch

F64 = torch.float64
# When set, every value that a bfloat16 implementation stores in bfloat16 (inputs and results of matrix products,
# activations, cached rows) is rounded to bfloat16 here as well.  The distance between that run and the exact one is
# the size of rounding noise for a given model and input: tests bound a bfloat16 run by a small multiple of it.
ROUND_BF16 = False


def _r(x):
    return x.to(torch.bfloat16).to(F64) if ROUND_BF16 else x


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is ONE number g for all coordinates."""
    return unit_rms(x, eps) * g


def vector_norm(x, w, eps):
    """RMS norm with a weight per coordinate."""
    return unit_rms(x, eps) * w


def token_shift(h, mu, before):
    """h [T][W]: row t becomes h_t + (h_{t-1} - h_t) * mu with the UNSHIFTED h_{t-1}; `before` is the row that
    precedes row 0 (zeros at the start of a sequence)."""
    prev = torch.cat([before.view(1, -1), h[:-1]], 0)
    return h + (prev - h) * mu


def rotate_pairs(x, pos, base, dims):
    """Rotary position on the first `dims` coordinates of the last axis of x [T][...][d], pairs (2i, 2i+1), angle
    pos * base^(-2i/dims); the remaining coordinates pass through."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = pos.to(F64).view(T, *([1] * (x.dim() - 1))) * base ** (-2.0 * i / dims)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * torch.cos(ang) - v * torch.sin(ang)
    out[..., 1:dims:2] = v * torch.cos(ang) + u * torch.sin(ang)
    return out


def sink_softmax(scores, sink):
    """softmax over the last axis of `scores` (-inf = masked) whose denominator also holds exp(sink); the sink has no
    value, so the weights sum to less than one."""
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def latent_kv(h, pos, w, pre, mx, eps):
    """The two things a latent-attention layer with its own down projection stores per token: the normed latent
    c [T][R] and the rotated key part shared by all heads kr [T][dr]."""
    R, dr = mx["kv_rank"], mx["rot_dim"]
    d = _r(h @ w[pre + "dkv"].to(F64).T)
    c = _r(vector_norm(d[:, :R], w[pre + "dkv.norm"].to(F64), eps))
    kr = _r(rotate_pairs(d[:, R:R + dr], pos, mx["rot"]["base"], mx["rot"]["dims"]))
    return c, kr


def latent_attention(h, pos, c_all, kr_all, w, pre, mx):
    """h [T][W] at positions pos [T]; c_all / kr_all hold the latents and rotated key parts of positions 0 .. max(pos)
    of the sequence (this layer's own, or the layer's it borrows them from).  Keys and values are expanded per head
    from the latent; softmax with a per-head sink; a per-head sigmoid gate read from h; then the output projection."""
    T = h.shape[0]
    H, dn, dr, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = _r(h @ w[pre + "q"].to(F64).T).view(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_pairs(q[..., dn:], pos, mx["rot"]["base"], mx["rot"]["dims"])
    S = c_all.shape[0]
    kn = _r(c_all @ w[pre + "uk"].to(F64).T).view(S, H, dn)
    v = _r(c_all @ w[pre + "uv"].to(F64).T).view(S, H, dv)
    s = (torch.einsum("thd,shd->hts", qn, kn) + torch.einsum("thd,sd->hts", qr, kr_all)) * mx["scale"]
    seen = torch.arange(S).view(1, 1, S) <= pos.view(1, T, 1)
    s = s.masked_fill(~seen, -math.inf)
    p = sink_softmax(s, w[pre + "sink"].to(F64).view(H, 1, 1))
    o = torch.einsum("hts,shd->thd", p, v)
    gate = torch.sigmoid(_r(h @ w[pre + "g"].to(F64).T))          # [T][H]
    o = _r(o * gate.unsqueeze(-1))
    return _r(o.reshape(T, H * dv) @ w[pre + "o"].to(F64).T)


def clipped_glu_expert(h, w, pre, limit):
    """g = min(G h, limit), u = clamp(U h, +-limit), y = g sigmoid(1.702 g) (u + 1), out = D y."""
    g = torch.clamp(_r(h @ w[pre + "gate"].to(F64).T), max=limit)
    u = torch.clamp(_r(h @ w[pre + "up"].to(F64).T), -limit, limit)
    return _r(_r(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].to(F64).T)


def route(h, w_router, top):
    """softmax over ALL experts, then the `top` largest scores as they are (no renormalisation) -> (weights, indices)."""
    s = torch.softmax(h @ w_router.to(F64).T, -1)
    return torch.topk(s, top, dim=-1)


def mixture(h, w, pre, mlp):
    """Routed experts weighted by their scores, plus a shared expert for every token."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    h = _r(h)
    wt, idx = route(h, w[pre + "router"], top)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for e in range(E):
        y = clipped_glu_expert(h, w, f"{pre}e{e}.", mlp["expert"]["limit"])
        out += y * (wt * (idx == e)).sum(-1, keepdim=True)
    if mlp.get("shared"):
        out += clipped_glu_expert(h, w, pre + "shared.", mlp["shared"]["limit"])
    return out


def depth_average(streams, coef):
    """sum_j coef[j] * streams[j] over all layer results so far (streams[0] = the embedding output)."""
    return sum(coef[j] * streams[j] for j in range(len(streams)))


def forward(cfg, w, tokens, return_layers=False):
    """Whole sequence at once, no cache: tokens [T] -> logits [T][vocab] in float64 (and the stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    pos = torch.arange(T)
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"].to(F64)[tokens]
    streams, after, kv = [x], [], {}
    for i, layer in enumerate(cfg["layers"]):
        assert layer["type"] == "latent_attention"
        mx, pre = layer["mixer"], f"l{i}."
        h = _r(token_shift(x, w[pre + "shift"].to(F64), torch.zeros(x.shape[1], dtype=F64)))
        if "kv_from" in mx:
            c, kr = kv[mx["kv_from"]]
        else:
            c, kr = kv[i] = latent_kv(h, pos, w, pre + "mix.", mx, eps)
        a = latent_attention(h, pos, c, kr, w, pre + "mix.", mx)
        x = x + m * scalar_norm(a, w[pre + "norm1"].to(F64), eps)
        if layer.get("mlp"):
            assert layer["mlp"]["kind"] == "moe"
            x = x + m * scalar_norm(mixture(x, w, pre + "mlp.", layer["mlp"]), w[pre + "norm2"].to(F64), eps)
        streams.append(x)
        x = depth_average(streams, w[pre + "dwa"].to(F64))
        after.append(x)
    logits = _r(scalar_norm(x, w["final.norm"].to(F64), eps)) @ w["head"].to(F64).T
    return (logits, torch.stack(after)) if return_layers else logits


def rounding_noise(cfg, w, tokens, measure):
    """measure(run with bfloat16 roundings, exact run): how far rounding alone moves the logits of this input."""
    global ROUND_BF16
    exact = forward(cfg, w, tokens)
    ROUND_BF16 = True
    try:
        rounded = forward(cfg, w, tokens)
    finally:
        ROUND_BF16 = False
    return measure(rounded, exact)


def greedy(cfg, w, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence for every new token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq


# ----------------------------------------------------------------------------------------------- test models
def random_config(width=64, vocab=97, heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, n_layers=3, share=(None, 0, None),
                  experts=4, top=2, ff=24, shared_ff=20, limit=1.5, shared_limit=2.5, base=10000.0, eps=1e-5, mult=0.6,
                  no_mlp=()):
    """A small configuration in the checkpoint's config.json form; share[i] = j makes layer i borrow layer j's latents."""
    layers = []
    for i in range(n_layers):
        mx = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim}, "rot_dim": rot_dim,
              "scale": 1.0 / math.sqrt(dim + rot_dim), "vdim": vdim}
        if share[i] is not None:
            mx["kv_from"] = share[i]
        mlp = None if i in no_mlp else {
            "expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "top": top},
            "shared": {"ff": shared_ff, "limit": shared_limit}}
        layers.append({"mixer": mx, "mlp": mlp, "type": "latent_attention"})
    return {"architecture": "Bitipel", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab,
            "width": width}


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Seeded weights with every tensor of the design, scaled so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(dtype), "head": mat(cfg["vocab"], W),
         "final.norm": (1.0 + 0.1 * torch.randn((), generator=g)).to(dtype)}
    for i, layer in enumerate(cfg["layers"]):
        mx, p = layer["mixer"], f"l{i}."
        H, dn, dr, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
        w[p + "norm1"] = (1.0 + 0.2 * torch.randn((), generator=g)).to(dtype)
        w[p + "shift"] = torch.rand(W, generator=g).to(dtype)
        w[p + "dwa"] = (torch.randn(i + 2, generator=g) * 0.3 + (torch.arange(i + 2) == i + 1) * 0.8).to(dtype)
        w[p + "mix.q"] = mat(H * (dn + dr), W, 2.0)
        if "kv_from" not in mx:
            w[p + "mix.dkv"] = mat(R + dr, W, 2.0)
            w[p + "mix.dkv.norm"] = (1.0 + 0.2 * torch.randn(R, generator=g)).to(dtype)
        w[p + "mix.uk"] = mat(H * dn, R, 2.0)
        w[p + "mix.uv"] = mat(H * dv, R)
        w[p + "mix.sink"] = torch.randn(H, generator=g).to(dtype)
        w[p + "mix.g"] = mat(H, W, 2.0)
        w[p + "mix.o"] = mat(W, H * dv)
        if layer["mlp"]:
            mlp = layer["mlp"]
            w[p + "norm2"] = (1.0 + 0.2 * torch.randn((), generator=g)).to(dtype)
            w[p + "mlp.router"] = mat(mlp["router"]["experts"], W, 3.0)
            names = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                names.append(("shared.", mlp["shared"]["ff"]))
            for n, ff in names:
                w[p + "mlp." + n + "gate"] = mat(ff, W, 2.0)
                w[p + "mlp." + n + "up"] = mat(ff, W, 2.0)
                w[p + "mlp." + n + "down"] = mat(W, ff)
    return w


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw little-endian data)."""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, at = {}, [], 0
    for name, t in w.items():
        raw = t.contiguous().view(-1).view(torch.uint8).numpy().tobytes() if t.dim() else \
            t.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
