"""Plain, slow restatement of the Tadolix decoder in float64 torch on the CPU: one function per mechanism, written from
the equations alone.  It shares no code with the package: tests compare the framework's kernels, state manager and
scheduler against it.  Weights are a dict {tensor name: tensor} with the checkpoint's names, the configuration is the
dict that config.json holds.  Every function takes a WHOLE sequence from position 0: nothing is cached here.

Notation: W = model width, T = tokens, S = streams, H / G = query / key-value heads, d / dv = key / value size per head,
C = chunk size of the attention mask, Rw = width of a recurrence.  A linear weight is stored [out][in]: y = M @ x.
"""
import json
import math
import os
import struct

import torch

F64 = torch.float64
# When set, what a bfloat16 implementation stores in bfloat16 (inputs and results of matrix products, activations,
# cached keys and values) is rounded to bfloat16 here as well; the distance between that run and the exact one is the
# size of rounding noise for a given model and input.
ROUND_BF16 = False


def _r(x):
    return x.to(torch.bfloat16).to(F64) if ROUND_BF16 else x


def _w(w, name):
    return w[name].to(F64)


def linear(x, w, name, bias=None):
    y = _r(x) @ _w(w, name).T
    if bias is not None:
        y = y + _w(w, bias)
    return _r(y)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def sinusoid(T, W):
    """[T][W]: coordinate 2i = sin(p f_i), 2i+1 = cos(p f_i), f_i = 10000^(-2i/W)."""
    out = torch.zeros(T, W, dtype=F64)
    p = torch.arange(T, dtype=F64).view(T, 1)
    i = torch.arange((W + 1) // 2, dtype=F64)
    ang = p * 10000.0 ** (-2.0 * i / W)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)[:, : W // 2]
    return out


def embed(cfg, w, tokens):
    T, W = len(tokens), cfg["width"]
    x = _w(w, "embed")[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    return x + sinusoid(T, W)


def causal_conv(x, kernel, bias=None):
    """x [T][C], kernel [C][taps]: y_t = sum_j kernel[:, j] * x_(t - taps + 1 + j), zeros before row 0 (the last
    column meets the current row)."""
    T, taps = x.shape[0], kernel.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F64), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + kernel[:, j] * pad[j:j + T]
    if bias is not None:
        y = y + bias
    return y


def distance_bucket(n, B, D):
    """Row of the distance-bias table for distance n >= 0: one row per distance below B // 2, logarithmic steps up
    to distance D above, everything farther in the last row."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def chunk_attention(h, w, pre, a, eps):
    """The attention branch: grouped heads, unit-RMS queries and keys, soft-capped scores, a learned bias per distance
    bucket and head, keys of the query's own chunk only, softmax, a sigmoid gate per output coordinate."""
    T = h.shape[0]
    H, G, d, dv, C = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
    q = linear(h, w, pre + "q").view(T, H, d)
    k = linear(h, w, pre + "k").view(T, G, d)
    v = linear(h, w, pre + "v").view(T, G, dv)
    gate = torch.sigmoid(linear(h, w, pre + "g"))
    q, k = unit_rms(q, eps), _r(unit_rms(k, eps))
    rel = _w(w, pre + "rel")
    B, cap = rel.shape[0], a["softcap"]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        kv = hd // (H // G)
        for i in range(T):
            lo = (i // C) * C
            s = (k[lo:i + 1, kv] @ q[i, hd]) * a["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s + torch.stack([rel[distance_bucket(i - j, B, a["bias_max"]), hd] for j in range(lo, i + 1)])
            p = torch.softmax(s, 0)
            out[i, hd] = p @ v[lo:i + 1, kv]
    return linear(out.reshape(T, H * dv) * gate, w, pre + "o")


def min_gru(h, w, pre):
    """The recurrent branch beside the attention: S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0, gates from the current
    token alone; c = u + 1/2 for u >= 0 and sigmoid(u) below."""
    z = torch.sigmoid(linear(h, w, pre + "z", pre + "z.b"))
    u = linear(h, w, pre + "x", pre + "x.b")
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = linear(h, w, pre + "g")
    S = torch.zeros(z.shape[1], dtype=F64)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        rows.append(S)
    S = torch.stack(rows)
    return linear(S * (g * torch.sigmoid(g)), w, pre + "o")


def parallel_mixer(h, w, pre, m, eps):
    return m["left_scale"] * chunk_attention(h, w, pre + "left.", m["left"], eps) + m["right_scale"] * min_gru(h, w, pre + "right.")


def rglru_mixer(h, w, pre, m):
    """A gelu branch times a real-gated linear recurrence over a short convolution of the other branch; the gates come
    from block-diagonal matrices."""
    T, nb = h.shape[0], m["blocks"]
    y = gelu_tanh(linear(h, w, pre + "y", pre + "y.b"))
    u = _r(causal_conv(linear(h, w, pre + "x", pre + "x.b"), _w(w, pre + "conv"), _w(w, pre + "conv.b")))
    Rw = u.shape[1]
    ub = u.view(T, nb, Rw // nb)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", _w(w, pre + "ra"), ub) + _w(w, pre + "ra.b")).reshape(T, Rw)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", _w(w, pre + "ri"), ub) + _w(w, pre + "ri.b")).reshape(T, Rw)
    log_a = -8.0 * r * torch.nn.functional.softplus(_w(w, pre + "lam"))
    a = torch.exp(log_a)
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(Rw, dtype=F64)
    rows = []
    for t in range(T):
        S = a[t] * S + b[t]
        rows.append(S)
    return linear(torch.stack(rows) * y, w, pre + "o")


def dense_ff(h, w, pre):
    return linear(gelu_tanh(linear(h, w, pre + "gate")) * linear(h, w, pre + "up"), w, pre + "down")


def layer_runs(cfg):
    """Order in which the layers run: the looped span `times` times in a row, every pass with state of its own."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T][vocab] of a whole sequence; with return_layers also the sum of the streams after every layer run."""
    eps, S = cfg["norm"]["eps"], cfg.get("streams")
    x0 = embed(cfg, w, tokens)
    xs = [x0.clone() for _ in range(S or 1)]
    after = []
    for li in layer_runs(cfg):
        lay, p = cfg["layers"][li], f"l{li}."
        for q in (1, 2):
            if q == 2 and not lay.get("mlp"):
                continue
            if S:
                cin, cout, cmix = _w(w, f"{p}hc{q}.in"), _w(w, f"{p}hc{q}.out"), _w(w, f"{p}hc{q}.mix")
                u = sum(cin[s] * xs[s] for s in range(S))
            else:
                u = xs[0]
            h = offset_norm(u, _w(w, f"{p}norm{q}"), eps)
            if q == 1:
                if cfg.get("canon"):
                    h = h + _r(causal_conv(_r(h), _w(w, p + "canon1")))
                if lay["type"] == "parallel":
                    y = parallel_mixer(h, w, p + "mix.", lay["mixer"], eps)
                elif lay["type"] == "rglru":
                    y = rglru_mixer(h, w, p + "mix.", lay["mixer"])
                else:
                    raise ValueError(lay["type"])
            else:
                assert lay["mlp"]["kind"] == "dense"
                y = dense_ff(h, w, p + "mlp.")
            if S:
                xs = [sum(cmix[s, t] * xs[s] for s in range(S)) + cout[t] * y for t in range(S)]
            else:
                xs = [xs[0] + y]
        after.append(sum(xs))
    x = sum(xs)
    logits = _r(offset_norm(x, _w(w, "final.norm"), eps)) @ _w(w, "head").T
    return (logits, torch.stack(after)) if return_layers else logits


def rounding_noise(cfg, w, tokens, measure):
    """measure(exact logits, logits of the run that rounds to bfloat16 wherever a bfloat16 implementation does)."""
    global ROUND_BF16
    exact = forward(cfg, w, tokens)
    ROUND_BF16 = True
    try:
        rounded = forward(cfg, w, tokens)
    finally:
        ROUND_BF16 = False
    return measure(exact, rounded)


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


# ------------------------------------------------------------------------------------------------ test models
def attention_layer(heads=4, kv_heads=2, dim=8, vdim=12, chunk=8, rows=6, bias_max=20, scale=0.3, softcap=5.0, right=24,
                    left_scale=0.7, right_scale=1.1, ff=40):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                               "bias_max": bias_max, "scale": scale, "softcap": softcap},
                      "left_scale": left_scale, "right": {"width": right}, "right_scale": right_scale, "_rel_rows": rows},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def recurrent_layer(width=24, blocks=3, conv=3, ff=0):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, width=32, vocab=61, streams=2, taps=3, loop=None, eps=1e-5, emb_scale=3.0):
    cfg = {"architecture": "Tadolix", "embedding": {"scale": emb_scale}, "layers": layers, "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if streams:
        cfg["streams"] = streams
    if taps:
        cfg["canon"] = {"taps": taps}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Every tensor the configuration names, seeded, sized so that each mechanism moves the logits: recurrences that
    remember for tens of tokens, distance biases of the order of the scores."""
    g = torch.Generator().manual_seed(seed)
    W, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")

    def mat(o, i, s=1.0):
        return torch.randn(o, i, generator=g, dtype=torch.float32) * (s / math.sqrt(i))

    def vec(n, mean=0.0, s=1.0):
        return mean + s * torch.randn(n, generator=g, dtype=torch.float32)

    w = {"embed": vec((V, W), 0.0, 0.5), "head": mat(V, W, 2.0), "final.norm": vec(W, 0.0, 0.2)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        w[p + "norm1"] = vec(W, 0.0, 0.2)
        if cfg.get("canon"):
            w[p + "canon1"] = vec((W, cfg["canon"]["taps"]), 0.0, 0.4)
        qs = (1, 2) if lay.get("mlp") else (1,)
        if S:
            for q in qs:
                w[f"{p}hc{q}.in"] = vec(S, 1.0 / S, 0.2)
                w[f"{p}hc{q}.out"] = vec(S, 0.6, 0.3)
                w[f"{p}hc{q}.mix"] = torch.eye(S) * 0.8 + vec((S, S), 0.0, 0.15)
        if lay["type"] == "parallel":
            a, Rw = m["left"], m["right"]["width"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            w[q + "q"], w[q + "k"], w[q + "v"] = mat(H * d, W, 2.0), mat(G * d, W, 2.0), mat(G * dv, W, 2.0)
            w[q + "g"], w[q + "o"] = mat(H * dv, W, 2.0), mat(W, H * dv, 1.5)
            w[q + "rel"] = vec((m.get("_rel_rows", 8), H), 0.0, 1.0)
            r = p + "mix.right."
            w[r + "z"], w[r + "x"], w[r + "g"], w[r + "o"] = mat(Rw, W, 2.0), mat(Rw, W, 2.0), mat(Rw, W, 2.0), mat(W, Rw, 1.5)
            w[r + "z.b"], w[r + "x.b"] = vec(Rw, -2.0, 1.0), vec(Rw, 0.0, 0.5)
        else:
            Rw, nb, q = m["width"], m["blocks"], p + "mix."
            w[q + "y"], w[q + "x"], w[q + "o"] = mat(Rw, W, 2.0), mat(Rw, W, 2.0), mat(W, Rw, 3.0)
            w[q + "y.b"], w[q + "x.b"] = vec(Rw, 0.0, 0.3), vec(Rw, 0.0, 0.3)
            w[q + "conv"], w[q + "conv.b"] = vec((Rw, m["conv"]), 0.3, 0.4), vec(Rw, 0.0, 0.2)
            bw = Rw // nb
            w[q + "ra"] = torch.randn(nb, bw, bw, generator=g) * (1.0 / math.sqrt(bw))
            w[q + "ri"] = torch.randn(nb, bw, bw, generator=g) * (1.0 / math.sqrt(bw))
            w[q + "ra.b"], w[q + "ri.b"] = vec((nb, bw), -1.0, 1.0), vec((nb, bw), 0.5, 1.0)
            w[q + "lam"] = vec(Rw, -3.0, 1.0)
        if lay.get("mlp"):
            ff = lay["mlp"]["ff"]
            w[p + "norm2"] = vec(W, 0.0, 0.2)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W, 2.0), mat(ff, W, 2.0), mat(W, ff, 1.5)
    return {k: v.to(dtype) for k, v in w.items()}


def clean_config(cfg):
    """The configuration without the keys that only random_weights reads (what a checkpoint's config.json holds)."""
    out = json.loads(json.dumps(cfg))
    for lay in out["layers"]:
        lay["mixer"].pop("_rel_rows", None)
    return out


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw data) in `folder`."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(clean_config(cfg), f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, at = {}, [], 0
    for name, t in w.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
