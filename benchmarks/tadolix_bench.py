"""Prefill and decode throughput of Tadolix layers at sizes of real models (random weights), beside the Llama family at
equal size in bf16 (same width, vocabulary and layer count, heads of 128 with 4:1 grouping, a feed-forward sized so that
the weights per layer match), and the design's own kernels timed alone against their roofline, each beside the like
kernel of the framework's other models.  `python bench.py --workload tadolix-layers` prints the result as one JSON line;
this file is the measurement.

Timing: CUDA events on the launching stream after 3 warm-up runs; model inputs and weights exceed L2, the kernel-alone
timings write a 256 MB buffer between runs.  Rooflines: measured copy bandwidth and cuBLAS bf16 rate of
MEASURED_PEAKS.json ("of measured"), or 6.65 TB/s and 1590 TF/s ("of fallback").
"""
import ctypes
import json
import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from benchmarks.bitipel_bench import peaks, timed  # noqa: E402


def llama_equal(cfg, weight_bytes, device):
    """The Llama family with the width, vocabulary and layer count of a Tadolix configuration and as many weight bytes
    in its layers, bf16."""
    from torchao_fork_b200._models.llama.model import ModelArgs, Transformer
    W, nl = cfg.width, cfg.n_layer
    heads, kv = W // 128, max(1, W // 512)
    attn = (W + 2 * kv * 128 + W) * W
    layers_bytes = weight_bytes - cfg.vocab_size * W * 2          # without the head
    inter = max(256, int(round((layers_bytes / 2 / nl - attn) / (3 * W) / 256)) * 256)
    args = ModelArgs(block_size=8192, vocab_size=cfg.vocab_size, n_layer=nl, n_head=heads, n_local_heads=kv, dim=W,
                     intermediate_size=inter, rope_base=500000)
    torch.manual_seed(0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            m = Transformer(args).eval()
    finally:
        torch.set_default_dtype(old)
    return m


def model_numbers(name, prompt_len, decode_ctx, decode_steps):
    """prefill tokens/s of a prompt and decode tokens/s (batch 1, CUDA graph) for Tadolix `name` and the Llama of equal size."""
    from torchao_fork_b200._models.llama.generate import Generator, prefill
    from torchao_fork_b200._models.tadolix import Tadolix, tadolix_configs
    dev = torch.device("cuda")
    out = {}
    cfg = tadolix_configs[name]()
    tadolix_bytes = None
    for fam in ("tadolix", "llama"):
        model = Tadolix.from_name(name, dev) if fam == "tadolix" else llama_equal(cfg, tadolix_bytes, dev)
        if fam == "tadolix":
            tadolix_bytes = model.weight_bytes(True)
        S = max(prompt_len, decode_ctx + decode_steps + 8)
        gen = Generator(model, 1, S, temperature=0.0, top_k=None)
        prompt = torch.randint(0, cfg.vocab_size, (1, prompt_len), device=dev)
        pos = torch.arange(prompt_len, device=dev, dtype=torch.int32)
        with torch.no_grad():
            ms_prefill = timed(lambda: prefill(model, prompt, pos, temperature=0.0, top_k=None), iters=3, warmup=2)
            prefill(model, prompt[:, :decode_ctx], pos[:decode_ctx], temperature=0.0, top_k=None)

            def decode():
                gen.engine.set_state(torch.zeros(1, dtype=torch.int64, device=dev), decode_ctx)
                gen.decode_tokens(decode_steps)
            ms_decode = timed(decode, iters=3, warmup=2) / decode_steps
        wb = tadolix_bytes if fam == "tadolix" else sum(p.numel() * p.element_size() for n, p in model.named_parameters()
                                                       if "tok_embeddings" not in n)
        out[fam] = {"prefill_tokens": prompt_len, "prefill_ms": round(ms_prefill, 3), "prefill_tok_per_s": round(prompt_len / ms_prefill * 1e3, 1),
                    "decode_context": decode_ctx, "decode_ms_per_token": round(ms_decode, 4), "decode_tok_per_s": round(1e3 / ms_decode, 1),
                    "decode_weight_gbs": round(wb / ms_decode / 1e6, 1),
                    "launches_per_decode_step": int(getattr(gen.engine, "launches_per_step", 0)), "weight_gb": round(wb / 1e9, 3)}
        if fam == "tadolix":
            out[fam]["state_bytes_per_sequence"] = model.state_bytes_per_sequence()
        del gen, model
        torch.cuda.empty_cache()
    return out


def kernel_numbers(name, prompt_len):
    """The design's kernels alone, at one layer's shapes, with the like kernel of another family beside each."""
    from torchao_fork_b200 import _lib
    from torchao_fork_b200._models.tadolix import tadolix_configs
    from torchao_fork_b200._models.tadolix.step import SCAN_TILE, chunk_tiles, scan_tiles
    hbm, tf, src = peaks()
    L = _lib.lm()
    dev = torch.device("cuda")
    st = torch.cuda.current_stream().cuda_stream
    cfg = tadolix_configs[name]()
    par = next(la for la in cfg.layers if la.type == "parallel").mixer
    rec = next(la for la in cfg.layers if la.type == "rglru").mixer
    a, W, S = par.left, cfg.width, max(1, cfg.streams)
    H, G, d, dv, C = a.heads, a.kv_heads, a.dim, a.vdim, a.chunk
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    res = {"roofline_source": src, "hbm_gbs": hbm, "bf16_tflops": tf}
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    i32 = lambda v: torch.as_tensor(np.asarray(v, np.int32)).to(dev)
    n = prompt_len

    # ---- attention of a whole prompt (tensor-core form): rows x visible keys x heads x (d + dv) multiply-adds are the
    # algorithm; the kernel issues d + 3 dv of them (the fp32 weights enter as three bf16 parts)
    pos_np = np.arange(n)
    slot, pos, back = i32(np.zeros(n)), i32(pos_np), i32(pos_np)
    ahead = i32(pos_np[::-1].copy())
    tr = ctypes.c_int()
    L.ao_lm_chunk_attention_prompt_plan(0, H, G, d, dv, ctypes.byref(tr))
    qn = torch.randn(n, H, d, **f32)
    kn, vn = torch.randn(n, G, d, **bf), torch.randn(n, G, dv, **bf)
    ring_k, ring_v = torch.randn(1, C, G, d, **bf), torch.randn(1, C, G, dv, **bf)
    gate = torch.randn(n, H * dv, **f32)
    bias = torch.randn(H, C, **f32)
    out = torch.empty(n, H * dv, **bf)
    pairs = sum((p % C) + 1 for p in range(n))
    if tr.value:
        f, c = chunk_tiles(np.array([0]), np.array([n]), pos_np, tr.value, C)
        tf_, tc_ = i32(f), i32(c)

        def attend():
            _lib.lm_check(L.ao_lm_chunk_attention_prompt(
                qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), 0, gate.data_ptr(), H * dv,
                bias.data_ptr(), C, slot.data_ptr(), pos.data_ptr(), back.data_ptr(), tf_.data_ptr(), tc_.data_ptr(), len(f), H, G, d,
                dv, C, a.scale, a.softcap, 1.0, out.data_ptr(), H * dv, st), "chunk_attention_prompt")
        ms = timed(attend, flush=flush)
        flops, issued = 2.0 * pairs * H * (d + dv), 2.0 * pairs * H * (d + 3 * dv)
        res["chunk_attention_prefill"] = {"tokens": n, "chunk": C, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                          "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4),
                                          "issued_tflops": round(issued / ms / 1e9, 2), "frac_issued": round(issued / ms / 1e9 / tf, 4)}
    # the like kernels: the Bitipel family's prompt attention (same instruction path and exactness rules) over a prompt of
    # as many visible pairs per row as a chunk holds, and the library attention that the Llama prefill calls
    xt = ctypes.c_int()
    L.ao_lm_latent_attention_expanded_plan(0, 128, 64, 128, ctypes.byref(xt))
    if xt.value:
        m = C
        qn2, qr2 = torch.randn(H, m, 128, **bf), torch.randn(m, H, 64, **f32)
        kx, vx, kr = torch.randn(m, H * 128, **bf), torch.randn(m, H * 128, **bf), torch.randn(1, m, 64, **bf)
        sl2, ps2 = i32(np.zeros(m)), i32(np.arange(m))
        t2 = np.arange(0, m, xt.value)
        tf2, tc2, trow = i32(t2), i32(np.minimum(xt.value, m - t2)), i32(np.zeros(len(t2)))
        sink, gt2, o2 = torch.zeros(H, **bf), torch.ones(m, H, **f32), torch.empty(m, H * 128, **bf)

        def bitipel_attend():
            _lib.lm_check(L.ao_lm_latent_attention_expanded(
                qn2.data_ptr(), qr2.data_ptr(), kx.data_ptr(), vx.data_ptr(), kr.data_ptr(), 0, m, sl2.data_ptr(), ps2.data_ptr(),
                tf2.data_ptr(), tc2.data_ptr(), trow.data_ptr(), len(t2), m, H, 128, 64, 128, 0.05, sink.data_ptr(), gt2.data_ptr(),
                o2.data_ptr(), st), "latent_attention_expanded")
        ms = timed(bitipel_attend, flush=flush)
        p2 = m * (m + 1) / 2
        flops, issued = 2.0 * p2 * H * (128 + 64 + 128), 2.0 * p2 * H * (128 + 2 * 64 + 3 * 128)
        res["bitipel_attention_prefill_one_chunk"] = {"tokens": m, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                                      "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4),
                                                      "issued_tflops": round(issued / ms / 1e9, 2),
                                                      "frac_issued": round(issued / ms / 1e9 / tf, 4)}
    q = torch.randn(n // C, H, C, 128, **bf)
    ms = timed(lambda: torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True), flush=flush)
    flops = 2.0 * (n // C) * (C * (C + 1) / 2) * H * 256
    res["library_sdpa_same_pairs"] = {"tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                      "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4)}

    # ---- attention of one decoded token at the end of a chunk: the ring's rows are read once
    tg = ctypes.c_int()
    L.ao_lm_chunk_attention_plan(0, H, G, d, dv, ctypes.byref(tg))
    one, last = i32([0]), i32([C - 1])
    zero, cnt = i32([0]), i32([1])
    o1 = torch.empty(1, H * dv, **bf)

    ns = max(1, min(-(-C // 32), -(-2 * 148 // G), 64))      # what the step function picks for one sequence
    aws = torch.empty(max(16, int(L.ao_lm_chunk_attention_workspace_bytes(1, G, dv, ns))), dtype=torch.uint8, device=dev)

    def attend_decode():
        _lib.lm_check(L.ao_lm_chunk_attention(
            qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), 0, gate.data_ptr(), H * dv, bias.data_ptr(),
            C, one.data_ptr(), last.data_ptr(), zero.data_ptr(), zero.data_ptr(), cnt.data_ptr(), 1, H, G, d, dv, C, a.scale, a.softcap,
            1.0, ns, aws.data_ptr(), aws.numel(), o1.data_ptr(), H * dv, st), "chunk_attention")
    ms = timed(attend_decode, flush=flush)
    byts = C * G * (d + dv) * 2
    res["chunk_attention_decode"] = {"keys": C, "splits": ns, "us": round(ms * 1e3, 2), "cache_bytes": byts, "gbs": round(byts / ms / 1e6, 1),
                                     "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    core = _lib.lib()
    q1 = torch.randn(1, H, 128, **bf)
    kc, vc = torch.randn(1, G, C, 128, **bf), torch.randn(1, G, C, 128, **bf)
    ipos = torch.full((1,), C - 1, dtype=torch.int32, device=dev)
    lo = torch.empty(1, H, 128, **bf)
    lns = max(1, min(64, -(-C // 32)))
    lws = torch.zeros(max(16, int(core.ao_b200_decode_attention_workspace_bytes(1, H, lns))), dtype=torch.uint8, device=dev)

    def llama_decode_attention():
        _lib.check(core.ao_b200_decode_attention(q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), ipos.data_ptr(), lo.data_ptr(), 1, H, G,
                                                 128, C, 1.0 / math.sqrt(128), lns, lws.data_ptr(), lws.numel(), st), "decode_attention")
    ms = timed(llama_decode_attention, flush=flush)
    byts = 2 * G * C * 128 * 2
    res["llama_attention_decode"] = {"keys": C, "splits": lns, "us": round(ms * 1e3, 2), "cache_bytes": byts,
                                     "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}

    # ---- the recurrences over a whole prompt (three launches over 64-row tiles) and for one decoded token
    sf, sc, seg0, segn = scan_tiles(np.array([0]), np.array([n]), SCAN_TILE)
    d_sf, d_sc, d_s0, d_sn = i32(sf), i32(sc), i32(seg0), i32(segn)
    Rw = par.right_width
    proj = torch.randn(n, 3 * Rw, **f32)
    zb, xb = torch.zeros(Rw, **bf), torch.zeros(Rw, **bf)
    state = torch.zeros(1, Rw, **f32)
    ws = torch.empty(int(L.ao_lm_scan_workspace_bytes(len(sf), Rw)) // 4, **f32)
    so = torch.empty(n, Rw, **bf)

    def mingru(rows, tiles):
        f_, c_, nt, s0, sn, ns = tiles
        _lib.lm_check(L.ao_lm_mingru_scan(proj.data_ptr(), 3 * Rw, 0, Rw, 2 * Rw, zb.data_ptr(), xb.data_ptr(), 0, Rw, state.data_ptr(),
                                          slot.data_ptr(), pos.data_ptr(), back.data_ptr(), f_.data_ptr(), c_.data_ptr(), nt,
                                          s0.data_ptr() if s0 is not None else None, sn.data_ptr() if sn is not None else None, ns,
                                          ws.data_ptr(), 1.0, so.data_ptr(), Rw, st), "mingru_scan")
    ms = timed(lambda: mingru(n, (d_sf, d_sc, len(sf), d_s0, d_sn, 1)), flush=flush)
    byts = n * Rw * (3 * 4 + 2)       # the three projection columns read once, the result written once
    moved = n * Rw * (2 * 4 + 3 * 4 + 2)    # what the two passes over the rows move
    res["mingru_scan_prefill"] = {"tokens": n, "channels": Rw, "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                                  "frac_hbm": round(byts / ms / 1e6 / hbm, 4), "moved_gbs": round(moved / ms / 1e6, 1),
                                  "frac_hbm_moved": round(moved / ms / 1e6 / hbm, 4)}
    one_tile = (zero, cnt, 1, None, None, 0)
    ms = timed(lambda: mingru(1, one_tile), flush=flush)
    res["mingru_scan_decode"] = {"us": round(ms * 1e3, 2)}
    Rr, nb = rec.width, rec.blocks
    gates, u, ypre = torch.randn(nb, n, 2 * (Rr // nb), **f32), torch.randn(n, Rr, **f32), torch.randn(n, 2 * Rr, **f32)
    rb, lam = torch.zeros(Rr, **bf), torch.full((Rr,), -3.0, **bf)
    rstate, ro = torch.zeros(1, Rr, **f32), torch.empty(n, Rr, **bf)
    ws2 = torch.empty(int(L.ao_lm_scan_workspace_bytes(len(sf), Rr)) // 4, **f32)

    def rglru():
        _lib.lm_check(L.ao_lm_rglru_scan(gates.data_ptr(), n, Rr // nb, rb.data_ptr(), rb.data_ptr(), lam.data_ptr(), 8.0, u.data_ptr(),
                                         ypre.data_ptr(), 2 * Rr, rb.data_ptr(), 0, Rr, rstate.data_ptr(), None, 0, None, None, 0,
                                         slot.data_ptr(), pos.data_ptr(), back.data_ptr(), d_sf.data_ptr(), d_sc.data_ptr(), len(sf),
                                         d_s0.data_ptr(), d_sn.data_ptr(), 1, ws2.data_ptr(), ro.data_ptr(), st), "rglru_scan")
    ms = timed(rglru, flush=flush)
    byts = n * Rr * (4 * 4 + 2)
    moved = n * Rr * (3 * 4 + 4 * 4 + 2)
    res["rglru_scan_prefill"] = {"tokens": n, "channels": Rr, "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                                 "frac_hbm": round(byts / ms / 1e6 / hbm, 4), "moved_gbs": round(moved / ms / 1e6, 1),
                                 "frac_hbm_moved": round(moved / ms / 1e6 / hbm, 4)}

    # ---- the stream kernels over a prompt: read-out + norm (reads S fp32 rows, writes one), write-back (reads S + 1, writes S),
    # and the mixer's convolution (reads a row and its taps - 1 neighbours from cache, writes bf16)
    x = torch.randn(n, S, W, **f32)
    y, hn, h = torch.randn(n, W, **f32), torch.empty(n, W, **f32), torch.empty(n, W, **bf)
    cin, wn, mix = torch.ones(S, **bf), torch.zeros(W, **bf), torch.eye(S, **bf)

    def norm():
        _lib.lm_check(L.ao_lm_streams_norm(x.data_ptr(), None, n, S, W, cin.data_ptr(), wn.data_ptr(), 0, 1.0, 1e-6, hn.data_ptr(), None,
                                           st), "streams_norm")
    ms = timed(norm, flush=flush)
    byts = n * W * 4 * (S + 1)
    res["streams_norm_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}

    def update():
        _lib.lm_check(L.ao_lm_streams_update(x.data_ptr(), y.data_ptr(), 1, n, S, W, mix.data_ptr(), cin.data_ptr(), 0, None, None, 0,
                                             None, None, None, st), "streams_update")
    ms = timed(update, flush=flush)
    byts = n * W * 4 * (2 * S + 1)
    res["streams_update_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    taps = max(2, cfg.canon_taps)
    kern, cstate = torch.randn(W, taps, **bf), torch.zeros(1, taps - 1, W, **f32)

    def conv():
        _lib.lm_check(L.ao_lm_causal_conv(hn.data_ptr(), W, None, n, W, taps, kern.data_ptr(), None, 0, 1, cstate.data_ptr(),
                                          slot.data_ptr(), pos.data_ptr(), back.data_ptr(), None, h.data_ptr(), st), "causal_conv")
    ms = timed(conv, flush=flush)
    byts = n * W * (4 + 2)
    res["causal_conv_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    # the like kernel: the Bitipel family's residual add + norm + average of three earlier results over as many rows
    xin, yb = torch.randn(n, W, **f32), torch.randn(n, W, **bf)
    streams = torch.randn(4, n, W, **f32)
    g1, coef, avg = torch.ones(1, **bf), torch.ones(4, **bf), torch.empty(n, W, **f32)

    def resid():
        _lib.lm_check(L.ao_lm_residual_norm(xin.data_ptr(), yb.data_ptr(), 0, g1.data_ptr(), 0, 0.7, 1e-5, n, W, streams[3].data_ptr(), None,
                                            None, streams.data_ptr(), 3, n * W, coef.data_ptr(), avg.data_ptr(), None, st), "residual_norm")
    ms = timed(resid, flush=flush)
    byts = n * W * (4 + 2 + 3 * 4 + 2 * 4)
    res["bitipel_residual_norm_average_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                                                    "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    return res


def run(sizes=("Tadolix-2k", "Tadolix-4k"), prompt_len=2048, decode_ctx=1536, decode_steps=64):
    out = {"metric": "tadolix_layers_prefill_decode", "dtype": "bf16", "data": "synthetic", "n_gpus": 1, "sizes": {}}
    for name in sizes:
        out["sizes"][name] = {"models": model_numbers(name, prompt_len, decode_ctx, decode_steps),
                              "kernels": kernel_numbers(name, prompt_len)}
    return out


if __name__ == "__main__":
    print(json.dumps(run()))
