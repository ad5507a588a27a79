"""Prefill and decode throughput of Bitipel layers at sizes of real models (random weights), beside the Llama family at
equal size in bf16 (same width, heads of 128, as many layers, a feed-forward as wide as the experts a token uses), and
the design's own kernels timed alone against their roofline.  `python bench.py --workload bitipel-layers` prints the
result as one JSON line; this file is the measurement.

Timing: CUDA events on the launching stream after 3 warm-up runs; model inputs and weights exceed L2, the kernel-alone
timings write a 256 MB buffer between runs.  Rooflines: measured copy bandwidth and cuBLAS bf16 rate of
MEASURED_PEAKS.json ("of measured"), or 6.65 TB/s and 1590 TF/s ("of fallback").
"""
import ctypes
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        p = json.load(open(pk))
        return float(p.get("hbm_gbs", 6650.0)), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def timed(fn, iters=5, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def llama_equal(cfg, device):
    """The Llama family at the size of a Bitipel configuration, bf16."""
    from torchao_fork_b200._models.llama.model import ModelArgs, Transformer
    f = cfg.layers[0].mlp
    args = ModelArgs(block_size=8192, vocab_size=cfg.vocab_size, n_layer=cfg.n_layer, n_head=cfg.width // 128,
                     n_local_heads=max(1, cfg.width // 512), dim=cfg.width, intermediate_size=f.top * f.ff + f.shared_ff,
                     rope_base=500000)
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
    """prefill tokens/s of a prompt and decode tokens/s (batch 1, CUDA graph) for Bitipel `name` and the Llama of equal size."""
    from torchao_fork_b200._models.bitipel import Bitipel, bitipel_configs
    from torchao_fork_b200._models.llama.generate import Generator, prefill
    dev = torch.device("cuda")
    out = {}
    cfg = bitipel_configs[name]()
    for fam in ("bitipel", "llama"):
        model = Bitipel.from_name(name, dev) if fam == "bitipel" else llama_equal(cfg, dev)
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
        out[fam] = {"prefill_tokens": prompt_len, "prefill_ms": round(ms_prefill, 3), "prefill_tok_per_s": round(prompt_len / ms_prefill * 1e3, 1),
                    "decode_context": decode_ctx, "decode_ms_per_token": round(ms_decode, 4), "decode_tok_per_s": round(1e3 / ms_decode, 1),
                    "launches_per_decode_step": int(getattr(gen.engine, "launches_per_step", 0)),
                    "weight_gb": round((model.weight_bytes(True) if fam == "bitipel" else
                                        sum(p.numel() * p.element_size() for n, p in model.named_parameters() if "tok_embeddings" not in n)) / 1e9, 3)}
        del gen, model
        torch.cuda.empty_cache()
    return out


def kernel_numbers(name, prompt_len, decode_ctx):
    """The design's kernels alone, at one layer's shapes, with the Llama family's like kernel beside each."""
    from torchao_fork_b200 import _lib
    from torchao_fork_b200._models.bitipel import bitipel_configs
    hbm, tf, src = peaks()
    L = _lib.lm()
    dev = torch.device("cuda")
    st = torch.cuda.current_stream().cuda_stream
    cfg = bitipel_configs[name]()
    a, f, W = cfg.layers[0].mixer, cfg.layers[0].mlp, cfg.width
    H, R, dr = a.heads, a.kv_rank, a.rot_dim
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    res = {"roofline_source": src, "hbm_gbs": hbm, "bf16_tflops": tf}
    bf = dict(dtype=torch.bfloat16, device=dev)
    tt = ctypes.c_int()
    L.ao_lm_latent_attention_plan(0, H, R, dr, ctypes.byref(tt))

    def attention(n, first_pos, n_split):
        S = first_pos + n
        c, kr = torch.randn(1, S, R, **bf), torch.randn(1, S, dr, **bf)
        qa, qr = torch.randn(H, n, R, device=dev), torch.randn(n, H, dr, device=dev)
        slot = torch.zeros(n, dtype=torch.int32, device=dev)
        pos = torch.arange(first_pos, S, dtype=torch.int32, device=dev)
        tfst = torch.arange(0, n, tt.value, dtype=torch.int32, device=dev)
        tcnt = torch.clamp(n - tfst, max=tt.value).int()
        sink, gate = torch.zeros(H, **bf), torch.ones(n, H, device=dev)
        out = torch.empty(n, H, R, **bf)
        ws = torch.empty(max(16, int(L.ao_lm_latent_attention_workspace_bytes(n, H, R, n_split))), dtype=torch.uint8, device=dev)

        def run():
            _lib.lm_check(L.ao_lm_latent_attention(qa.data_ptr(), qr.data_ptr(), c.data_ptr(), kr.data_ptr(), 0, S, slot.data_ptr(),
                                                   pos.data_ptr(), tfst.data_ptr(), tcnt.data_ptr(), tfst.numel(), n, H, R, dr, a.scale,
                                                   sink.data_ptr(), gate.data_ptr(), S - 1, n_split, ws.data_ptr(), ws.numel(),
                                                   out.data_ptr(), st), "latent_attention")
        return timed(run, flush=flush)

    # prompt attention, expanded form: rows x visible keys x heads x (score: dn + dr, weighted sum: dv) multiply-adds are
    # the algorithm; the kernel issues (dn + 2 dr) + 3 dv of them (fp32 rotated queries in two bf16 parts, fp32 weights
    # in three).  The two GEMMs that up-project the cached latents into keys and values are timed beside it.
    n = prompt_len
    dn, dv = a.dim, a.vdim
    xt = ctypes.c_int()
    L.ao_lm_latent_attention_expanded_plan(0, dn, dr, dv, ctypes.byref(xt))
    if xt.value:
        qn, qr = torch.randn(H, n, dn, **bf), torch.randn(n, H, dr, device=dev)
        cl, kr = torch.randn(n, R, **bf), torch.randn(1, n, dr, **bf)
        ukx, uvx = torch.randn(H * dn, R, **bf) / math.sqrt(R), torch.randn(R, H * dv, **bf) / math.sqrt(R)
        kx, vx = torch.empty(n, H * dn, **bf), torch.empty(n, H * dv, **bf)
        slot = torch.zeros(n, dtype=torch.int32, device=dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        tfst = torch.arange(0, n, xt.value, dtype=torch.int32, device=dev)
        tcnt, trow = torch.clamp(n - tfst, max=xt.value).int(), torch.zeros_like(tfst)
        sink, gate = torch.zeros(H, **bf), torch.ones(n, H, device=dev)
        out = torch.empty(n, H * dv, **bf)

        def expand():
            torch.mm(cl, ukx.t(), out=kx)
            torch.mm(cl, uvx, out=vx)

        def expanded():
            _lib.lm_check(L.ao_lm_latent_attention_expanded(
                qn.data_ptr(), qr.data_ptr(), kx.data_ptr(), vx.data_ptr(), kr.data_ptr(), 0, n, slot.data_ptr(), pos.data_ptr(),
                tfst.data_ptr(), tcnt.data_ptr(), trow.data_ptr(), tfst.numel(), n, H, dn, dr, dv, a.scale, sink.data_ptr(),
                gate.data_ptr(), out.data_ptr(), st), "latent_attention_expanded")
        ms_x = timed(expand, flush=flush)
        ms = timed(expanded, flush=flush)
        pairs = n * (n + 1) / 2
        flops, issued = 2.0 * pairs * H * (dn + dr + dv), 2.0 * pairs * H * (dn + 2 * dr + 3 * dv)
        res["latent_attention_prefill"] = {
            "tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2), "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4),
            "issued_tflops": round(issued / ms / 1e9, 2), "frac_issued": round(issued / ms / 1e9 / tf, 4),
            "expand_gemms_ms": round(ms_x, 3)}
        del qn, qr, cl, kr, kx, vx, out
    # the folded form (what decoded tokens use) on the same prompt, for the record: (R + dr) + R multiply-adds per pair
    ms = attention(n, 0, 1)
    flops = 2.0 * (n * (n + 1) / 2) * H * (2 * R + dr)
    res["latent_attention_folded_on_a_prompt"] = {"tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2)}
    q = torch.randn(1, cfg.width // 128, n, 128, **bf)
    k = torch.randn(1, cfg.width // 128, n, 128, **bf)
    ms = timed(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, k, is_causal=True), flush=flush)
    flops = 2.0 * (n * (n + 1) / 2) * (cfg.width // 128) * 256
    res["llama_sdpa_prefill"] = {"tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                 "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4)}
    # one decoded token: the cached rows of the context are read once
    ns = max(1, min(-(-(decode_ctx + 1) // 32), -(-2 * 148 // -(-H // 16)), 64))   # what the decode engine picks
    ms = attention(1, decode_ctx, ns)
    byts = (decode_ctx + 1) * (R + dr) * 2
    res["latent_attention_decode"] = {"context": decode_ctx, "splits": ns, "us": round(ms * 1e3, 2), "cache_bytes": byts,
                                      "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    # the Llama family's decode attention at the same context: K and V rows of width / 512 heads of 128, read once
    core = _lib.lib()
    Hq, Hkv, S = W // 128, max(1, W // 512), decode_ctx + 1
    q1 = torch.randn(1, Hq, 128, **bf)
    kc, vc = torch.randn(1, Hkv, S, 128, **bf), torch.randn(1, Hkv, S, 128, **bf)
    ipos = torch.full((1,), decode_ctx, dtype=torch.int32, device=dev)
    o1 = torch.empty(1, Hq, 128, **bf)
    lns = max(1, min(64, -(-S // 32)))
    lws = torch.zeros(max(16, int(core.ao_b200_decode_attention_workspace_bytes(1, Hq, lns))), dtype=torch.uint8, device=dev)

    def llama_decode_attention():
        _lib.check(core.ao_b200_decode_attention(q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), ipos.data_ptr(), o1.data_ptr(), 1, Hq,
                                                 Hkv, 128, S, 1.0 / math.sqrt(128), lns, lws.data_ptr(), lws.numel(), st),
                   "decode_attention")
    ms = timed(llama_decode_attention, flush=flush)
    byts = 2 * Hkv * S * 128 * 2
    res["llama_attention_decode"] = {"context": decode_ctx, "splits": lns, "us": round(ms * 1e3, 2), "cache_bytes": byts,
                                     "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    # experts of one decoded token: top x (gate, up, down) matrices + the shared expert, read once
    tdt = torch.bfloat16
    x = torch.randn(1, W, **bf)
    wgu, wd = torch.randn(f.experts, 2 * f.ff, W, **bf), torch.randn(f.experts, W, f.ff, **bf)
    idx = torch.arange(f.top, dtype=torch.int32, device=dev).view(1, f.top)
    wt = torch.ones(1, f.top, device=dev)
    ya, ffo = torch.empty(f.top, f.ff, **bf), torch.empty(1, W, device=dev)

    def experts():
        _lib.lm_check(L.ao_lm_expert_gate_up(x.data_ptr(), wgu.data_ptr(), wgu.data_ptr() + f.ff * W * 2, 0, idx.data_ptr(), 1, f.top, W,
                                             f.ff, 2 * f.ff * W, f.limit, 1.702, ya.data_ptr(), st), "gate_up")
        _lib.lm_check(L.ao_lm_expert_down(ya.data_ptr(), wd.data_ptr(), 0, idx.data_ptr(), wt.data_ptr(), 1, f.top, W, f.ff, 0,
                                          ffo.data_ptr(), st), "down")
    ms = timed(experts, flush=flush)
    byts = f.top * 3 * f.ff * W * 2
    res["expert_gemv_decode"] = {"us": round(ms * 1e3, 2), "weight_bytes": byts, "gbs": round(byts / ms / 1e6, 1),
                                 "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    I = f.top * f.ff + f.shared_ff
    w13, w2 = torch.randn(2 * I, W, **bf), torch.randn(W, I, **bf)
    hmid = torch.randn(1, I, **bf)
    ms = timed(lambda: (torch.mm(x, w13.t()), torch.mm(hmid, w2.t())), flush=flush)
    byts = 3 * I * W * 2
    res["llama_bf16_ffn_gemv_decode"] = {"us": round(ms * 1e3, 2), "weight_bytes": byts, "gbs": round(byts / ms / 1e6, 1),
                                         "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    # residual add + scalar norm + depth average over 3 earlier results, prompt rows (reads 4 fp32 rows + y, writes 2 + a copy)
    xin, y = torch.randn(n, W, device=dev), torch.randn(n, W, **bf)
    streams = torch.randn(4, n, W, device=dev)
    g1, coef = torch.ones(1, **bf), torch.ones(4, **bf)
    avg = torch.empty(n, W, device=dev)

    def resid():
        _lib.lm_check(L.ao_lm_residual_norm(xin.data_ptr(), y.data_ptr(), 0, g1.data_ptr(), 0, 0.7, 1e-5, n, W, streams[3].data_ptr(), None,
                                            None, streams.data_ptr(), 3, n * W, coef.data_ptr(), avg.data_ptr(), None, st), "residual_norm")
    ms = timed(resid, flush=flush)
    byts = n * W * (4 + 2 * 2 + 3 * 4 + 2 * 4)
    res["residual_norm_average_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    from torchao_fork_b200._models.llama.model import RMSNorm
    norm = RMSNorm(W).to(dev, torch.bfloat16)
    xb = torch.randn(n, W, **bf)
    ms = timed(lambda: norm(xb + y), flush=flush)
    byts = n * W * 2 * 3
    res["llama_add_rmsnorm_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4),
                                        "note": "eager torch ops: several passes over the rows, algorithmic bytes counted once"}
    return res


def run(sizes=("Bitipel-2k", "Bitipel-4k"), prompt_len=2048, decode_ctx=1024, decode_steps=64):
    out = {"metric": "bitipel_layers_prefill_decode", "dtype": "bf16", "data": "synthetic", "n_gpus": 1, "sizes": {}}
    for name in sizes:
        out["sizes"][name] = {"models": model_numbers(name, prompt_len, decode_ctx, decode_steps),
                              "kernels": kernel_numbers(name, prompt_len, decode_ctx)}
    return out


if __name__ == "__main__":
    print(json.dumps(run()))
