"""Tadolix on the GPU against the float64 oracle (tests/tadolix_oracle.py): every mechanism's kernel alone, then the model
through the framework's step function, state manager, decode engine and Generator.  Configurations and weights are
made here; float32 runs are held to a tight bound (only summation order differs), bfloat16 runs to the rounding noise
of bf16 products."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import tadolix_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 1e-4
F64 = torch.float64


def _lm():
    from torchao_fork_b200 import _lib
    return _lib, _lib.lm()


def _st():
    return torch.cuda.current_stream().cuda_stream


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def _err(got, ref):
    """Root mean square of the difference (mean over the vocabulary taken off), relative to the reference's spread."""
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def _bf16_tol(cfg, w, toks):
    """A bfloat16 run may be 3 times as far from the exact logits as bfloat16 rounding alone moves them."""
    return 3.0 * O.rounding_noise(cfg, w, toks, _err)


def _model(cfg, w, dtype=torch.float32, slots=2, seq=4096):
    from torchao_fork_b200._models.tadolix import Tadolix, TadolixArgs
    m = Tadolix(TadolixArgs.from_dict(O.clean_config(cfg)), w, "cuda", dtype).eval()
    m.setup_caches(slots, seq)
    return m


def _tokens(cfg, n, seed=0):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _rows(segs):
    """[(slot, first position, rows)] -> per-row slot, pos, back, ahead on the device."""
    slot, pos, back, ahead = [], [], [], []
    for s, p0, c in segs:
        slot += [s] * c
        pos += list(range(p0, p0 + c))
        back += list(range(c))
        ahead += list(range(c - 1, -1, -1))
    return _i32(slot), _i32(pos), _i32(back), _i32(ahead)


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,S", [(32, 3), (33, 1), (70, 4)])
def test_embedding_scale_and_sinusoid_far_positions(dtype, W, S):
    lib, L = _lm()
    dt = lib.DT_F32 if dtype == torch.float32 else lib.DT_BF16
    cfg = {"width": W, "embedding": {"scale": 7.5}}
    table = torch.randn(11, W, generator=torch.Generator().manual_seed(0)).to(dtype)
    pos = [0, 1, 2, 63, 64, 4999, 70000]
    tok = [3, 0, 10, 3, 5, 1, 2]
    ref = table.double()[tok] * 7.5
    full = O.sinusoid(70001, W)
    ref = ref + full[pos]
    freq = (10000.0 ** (-2.0 * torch.arange((W + 1) // 2, dtype=F64) / W)).cuda()
    x = torch.empty(len(tok), S, W, device="cuda")
    td, kd, pd = table.cuda(), torch.tensor(tok, device="cuda"), _i32(pos)
    lib.lm_check(L.ao_lm_embed_sinusoid(td.data_ptr(), dt, kd.data_ptr(), pd.data_ptr(), len(tok), W, 7.5, freq.data_ptr(), S,
                                        x.data_ptr(), _st()), "embed_sinusoid")
    for s in range(S):
        assert torch.allclose(x[:, s].double().cpu(), ref, rtol=0, atol=2e-6), cfg


@pytest.mark.parametrize("S,W,coef", [(3, 40, True), (1, 33, False), (4, 64, False), (2, 257, True)])
def test_stream_read_out_and_norm(S, W, coef):
    lib, L = _lm()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(6, S, W, generator=g) * 3
    cin = torch.randn(S, generator=g).to(torch.bfloat16) if coef else None
    wn = (0.3 * torch.randn(W, generator=g)).to(torch.bfloat16)
    rows = [4, 0, 5]
    xd, cd, wd, rd = x.cuda(), (cin.cuda() if coef else None), wn.cuda(), _i32(rows)
    o32, o16 = torch.empty(3, W, device="cuda"), torch.empty(3, W, device="cuda", dtype=torch.bfloat16)
    lib.lm_check(L.ao_lm_streams_norm(xd.data_ptr(), rd.data_ptr(), 3, S, W, cd.data_ptr() if coef else None, wd.data_ptr(),
                                      lib.DT_BF16, 1.0, 1e-5, o32.data_ptr(), o16.data_ptr(), _st()), "streams_norm")
    u = sum((cin.double()[s] if coef else 1.0) * x.double()[:, s] for s in range(S))
    ref = O.offset_norm(u, wn.double(), 1e-5)[rows]
    assert torch.allclose(o32.double().cpu(), ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(o16.double().cpu(), ref, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("S,taps", [(3, 4), (1, 2), (4, 3)])
def test_stream_write_back_and_convolution_memory(S, taps):
    lib, L = _lm()
    W, g = 24, torch.Generator().manual_seed(2)
    # segments: slot 1 continues at position 9 with ONE row, slot 0 starts with 2 rows, slot 2 continues at 5 with 6 rows
    segs = [(1, 9, 1), (0, 0, 2), (2, 5, 6)]
    slot, pos, back, ahead = _rows(segs)
    n = 9
    x = torch.randn(n, S, W, generator=g)
    y = torch.randn(n, W, generator=g)
    mix, co = torch.randn(S, S, generator=g).to(torch.bfloat16), torch.randn(S, generator=g).to(torch.bfloat16)
    conv_in = torch.randn(n, W, generator=g)
    state0 = torch.randn(3, taps - 1, W, generator=g)
    xd, yd, md, cd, ci, sd = x.cuda(), y.cuda(), mix.cuda(), co.cuda(), conv_in.cuda(), state0.cuda()
    lib.lm_check(L.ao_lm_streams_update(xd.data_ptr(), yd.data_ptr(), lib.DT_F32, n, S, W, md.data_ptr(), cd.data_ptr(), lib.DT_BF16,
                                        ci.data_ptr(), sd.data_ptr(), taps, slot.data_ptr(), back.data_ptr(), ahead.data_ptr(),
                                        _st()), "streams_update")
    xf, mf, cf = x.double(), mix.double(), co.double()
    ref = torch.stack([sum(mf[s, t] * xf[:, s] for s in range(S)) + cf[t] * y.double() for t in range(S)], 1)
    assert torch.allclose(xd.double().cpu(), ref, rtol=1e-5, atol=1e-5)
    # memory = the last taps - 1 inputs of (old memory ++ the segment's rows)
    at = 0
    for s, p0, c in segs:
        hist = torch.cat([state0[s], conv_in[at:at + c]])[-(taps - 1):]
        assert torch.equal(sd[s].cpu(), hist), (s, c)
        at += c
    # identity write-back without weights: x + y
    x1 = x[:, :1].contiguous().cuda()
    lib.lm_check(L.ao_lm_streams_update(x1.data_ptr(), yd.data_ptr(), lib.DT_F32, n, 1, W, None, None, lib.DT_BF16, None, None, 0,
                                        None, None, None, _st()), "streams_update")
    assert torch.allclose(x1[:, 0].cpu(), x[:, 0] + y, atol=1e-6)


@pytest.mark.parametrize("taps,residual,bias", [(4, 1, False), (3, 0, True), (2, 0, True), (7, 1, False)])
def test_causal_convolution_in_portions_equals_the_whole_sequence(taps, residual, bias):
    lib, L = _lm()
    C, T, g = 37, 23, torch.Generator().manual_seed(3)
    x = torch.randn(T, C + 5, generator=g)            # the channels are columns 5 .. of a wider row
    kern = torch.randn(C, taps, generator=g).to(torch.bfloat16)
    ib = torch.randn(C, generator=g).to(torch.bfloat16) if bias else None
    ob = torch.randn(C, generator=g).to(torch.bfloat16) if bias else None
    v = x[:, 5:].double() + (ib.double() if bias else 0.0)
    ref = O.causal_conv(v, kern.double(), ob.double() if bias else None) + (v if residual else 0.0)
    state = torch.full((2, taps - 1, C), 777.0, device="cuda")      # a reused slot: stale rows must not be read at the start
    kd, ibd, obd = kern.cuda(), (ib.cuda() if bias else None), (ob.cuda() if bias else None)
    got, at = [], 0
    for c in [1, 2, 1, 5, 1, 1, 9, 3]:
        xs = x[at:at + c].contiguous().cuda()
        slot, pos, back, ahead = _rows([(1, at, c)])
        out = torch.empty(c, C, device="cuda")
        lib.lm_check(L.ao_lm_causal_conv(xs.data_ptr() + 20, C + 5, ibd.data_ptr() if bias else None, c, C, taps, kd.data_ptr(),
                                         obd.data_ptr() if bias else None, lib.DT_BF16, residual, state.data_ptr(), slot.data_ptr(),
                                         pos.data_ptr(), back.data_ptr(), out.data_ptr(), None, _st()), "causal_conv")
        # the memory is written by the kernel that closes the sublayer: here the stream write-back on a dummy stream
        dummy, zero = torch.zeros(c, 1, C, device="cuda"), torch.zeros(c, C, device="cuda")
        vin = (xs[:, 5:] + (ibd.float() if bias else 0.0)).contiguous()
        lib.lm_check(L.ao_lm_streams_update(dummy.data_ptr(), zero.data_ptr(), lib.DT_F32, c, 1, C, None, None, lib.DT_BF16,
                                            vin.data_ptr(), state.data_ptr(), taps, slot.data_ptr(), back.data_ptr(),
                                            ahead.data_ptr(), _st()), "streams_update")
        got.append(out.cpu())
        at += c
    assert at == T
    assert torch.allclose(torch.cat(got).double(), ref, rtol=1e-5, atol=1e-5)


def _scan_meta(segs, tile):
    from torchao_fork_b200._models.tadolix.step import scan_tiles
    starts = np.cumsum([0] + [c for _, _, c in segs[:-1]])
    counts = np.array([c for _, _, c in segs])
    f, c, s0, sn = scan_tiles(starts, counts, tile)
    return _i32(f.tolist()), _i32(c.tolist()), len(f), (None if s0 is None else _i32(s0.tolist())), (None if s0 is None else _i32(sn.tolist())), len(segs)


@pytest.mark.parametrize("tile", [64, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_minimal_gru_scan_in_portions_and_batches(tile, dtype):
    lib, L = _lm()
    dt = lib.DT_F32 if dtype == torch.float32 else lib.DT_BF16
    W, Rw, T, g = 16, 150, 41, torch.Generator().manual_seed(4)
    cfg = O.make_config([O.attention_layer(right=Rw)], width=W)
    w = {k: v.double() for k, v in O.random_weights(cfg, 5).items()}
    p = "l0.mix.right."
    w[p + "o"] = torch.eye(Rw, dtype=F64)
    h = [torch.randn(T, W, generator=g, dtype=F64), torch.randn(17, W, generator=g, dtype=F64)]
    ref = [O.min_gru(x, w, p) * 0.7 for x in h]
    proj = [torch.cat([x @ w[p + "z"].T, x @ w[p + "x"].T, x @ w[p + "g"].T], 1).float() for x in h]
    zb, xb = w[p + "z.b"].to(dtype).cuda(), w[p + "x.b"].to(dtype).cuda()
    state = torch.full((3, Rw), 55.0, device="cuda")
    got = [[], []]
    # steps: (sequence 0 rows, sequence 1 rows) in slots 2 and 0
    at = [0, 0]
    for c0, c1 in [(9, 1), (1, 1), (20, 2), (1, 13), (10, 0)]:
        segs, parts = [], []
        for k, (c, sl) in enumerate([(c0, 2), (c1, 0)]):
            if c:
                segs.append((sl, at[k], c))
                parts.append(proj[k][at[k]:at[k] + c])
        pj = torch.cat(parts).cuda()
        n = pj.shape[0]
        slot, pos, back, ahead = _rows(segs)
        tf, tc, nt, s0, sn, ns = _scan_meta(segs, tile)
        ws = torch.empty(max(1, int(L.ao_lm_scan_workspace_bytes(nt, Rw)) // 4), device="cuda")
        out = torch.zeros(n, Rw + 3, dtype=dtype, device="cuda")       # written at column 3 of a wider row
        lib.lm_check(L.ao_lm_mingru_scan(pj.data_ptr(), 3 * Rw, 0, Rw, 2 * Rw, zb.data_ptr(), xb.data_ptr(), dt, Rw, state.data_ptr(),
                                         slot.data_ptr(), pos.data_ptr(), back.data_ptr(), tf.data_ptr(), tc.data_ptr(), nt,
                                         s0.data_ptr() if s0 is not None else None, sn.data_ptr() if s0 is not None else None, ns,
                                         ws.data_ptr(), 0.7, out.data_ptr() + 3 * out.element_size(), Rw + 3, _st()), "mingru_scan")
        assert float(out[:, :3].abs().max()) == 0.0
        o, r = out[:, 3:].double().cpu(), 0
        for k, c in enumerate([c0, c1]):
            if c:
                got[k].append(o[r:r + c])
                r += c
                at[k] += c
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    for k in range(2):
        assert torch.allclose(torch.cat(got[k]), ref[k], **tol), k


@pytest.mark.parametrize("tile", [64, 3])
@pytest.mark.parametrize("Rw,nb,taps", [(24, 3, 3), (20, 1, 2), (16, 16, 4)])
def test_real_gated_recurrence_with_its_convolution_in_portions(tile, Rw, nb, taps):
    lib, L = _lm()
    W, T, g = 12, 30, torch.Generator().manual_seed(6)
    cfg = O.make_config([O.recurrent_layer(Rw, nb, taps)], width=W)
    w = {k: v.double() for k, v in O.random_weights(cfg, 7).items()}
    p = "l0.mix."
    w[p + "o"] = torch.eye(Rw, dtype=F64)
    h = torch.randn(T, W, generator=g, dtype=F64)
    ref = O.rglru_mixer(h, w, p, cfg["layers"][0]["mixer"])
    proj = torch.cat([h @ w[p + "y"].T, h @ w[p + "x"].T], 1).float()
    bw = Rw // nb
    dev = lambda t: t.float().contiguous().cuda()
    yb, xb, cw, cb, lam = dev(w[p + "y.b"]), dev(w[p + "x.b"]), dev(w[p + "conv"]), dev(w[p + "conv.b"]), dev(w[p + "lam"])
    rab, rib = dev(w[p + "ra.b"].reshape(-1)), dev(w[p + "ri.b"].reshape(-1))
    wg = torch.cat([w[p + "ra"].transpose(1, 2), w[p + "ri"].transpose(1, 2)], 2).float().cuda()
    state, cstate = torch.full((2, Rw), 9.0, device="cuda"), torch.full((2, taps - 1, Rw), 9.0, device="cuda")
    got, at = [], 0
    for c in [2, 1, 1, 11, 1, 14]:
        pj = proj[at:at + c].contiguous().cuda()
        segs = [(1, at, c)]
        slot, pos, back, ahead = _rows(segs)
        u = torch.empty(c, Rw, device="cuda")
        lib.lm_check(L.ao_lm_causal_conv(pj.data_ptr() + 4 * Rw, 2 * Rw, xb.data_ptr(), c, Rw, taps, cw.data_ptr(), cb.data_ptr(),
                                         lib.DT_F32, 0, cstate.data_ptr(), slot.data_ptr(), pos.data_ptr(), back.data_ptr(),
                                         u.data_ptr(), None, _st()), "causal_conv")
        gates = torch.bmm(u.view(c, nb, bw).transpose(0, 1), wg).contiguous()
        tf, tc, nt, s0, sn, ns = _scan_meta(segs, tile)
        ws = torch.empty(max(1, int(L.ao_lm_scan_workspace_bytes(nt, Rw)) // 4), device="cuda")
        out = torch.empty(c, Rw, device="cuda")
        lib.lm_check(L.ao_lm_rglru_scan(gates.data_ptr(), c, bw, rab.data_ptr(), rib.data_ptr(), lam.data_ptr(), 8.0, u.data_ptr(),
                                        pj.data_ptr(), 2 * Rw, yb.data_ptr(), lib.DT_F32, Rw, state.data_ptr(), pj.data_ptr() + 4 * Rw,
                                        2 * Rw, xb.data_ptr(), cstate.data_ptr(), taps, slot.data_ptr(), pos.data_ptr(), back.data_ptr(),
                                        tf.data_ptr(), tc.data_ptr(), nt, s0.data_ptr() if s0 is not None else None,
                                        sn.data_ptr() if s0 is not None else None, ns, ws.data_ptr(), out.data_ptr(), _st()), "rglru_scan")
        got.append(out.double().cpu())
        at += c
    assert torch.allclose(torch.cat(got), ref, rtol=2e-5, atol=2e-5)


def _attention_alone(a, w, h, cuts, dtype, slot=1, slots=3, tensor=False, n_split=1):
    """The three attention launches over `h` cut into portions, on a ring that starts full of stale rows; `tensor`
    picks the tensor-core form of the attention kernel."""
    lib, L = _lm()
    from torchao_fork_b200._models.tadolix.model import distance_bias_table
    from torchao_fork_b200._models.tadolix.step import chunk_tiles
    dt = lib.DT_F32 if dtype == torch.float32 else lib.DT_BF16
    p = "l0.mix.left."
    H, G, d, dv, C = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
    proj = torch.cat([h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T, h @ w[p + "g"].T], 1).float()
    ld = proj.shape[1]
    bias = distance_bias_table(w[p + "rel"].float().cuda(), a["bias_max"], C)
    ring_k = torch.full((slots, C, G, d), 3.0, dtype=dtype, device="cuda")
    ring_v = torch.full((slots, C, G, dv), -50.0, dtype=dtype, device="cuda")
    tr = __import__("ctypes").c_int()
    lib.lm_check((L.ao_lm_chunk_attention_prompt_plan if tensor else L.ao_lm_chunk_attention_plan)(
        dt, H, G, d, dv, __import__("ctypes").byref(tr)), "plan")
    assert tr.value > 0
    attend = L.ao_lm_chunk_attention_prompt if tensor else L.ao_lm_chunk_attention
    got, at = [], 0
    for c in cuts:
        pj = proj[at:at + c].contiguous().cuda()
        sl, pos, back, ahead = _rows([(slot, at, c)])
        qn = torch.empty(c, H, d, device="cuda")
        kn, vn = torch.empty(c, G, d, dtype=dtype, device="cuda"), torch.empty(c, G, dv, dtype=dtype, device="cuda")
        lib.lm_check(L.ao_lm_qk_prep(pj.data_ptr(), ld, 0, H * d, (H + G) * d, c, H, G, d, dv, 1e-6, dt, qn.data_ptr(), kn.data_ptr(),
                                     vn.data_ptr(), _st()), "qk_prep")
        f, k = chunk_tiles(np.array([0]), np.array([c]), np.arange(at, at + c), tr.value, C)
        tf, tc = _i32(f.tolist()), _i32(k.tolist())
        out = torch.zeros(c, H * dv + 2, dtype=dtype, device="cuda")
        args = (qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), dt,
                pj.data_ptr() + 4 * ((H + G) * d + G * dv), ld, bias.data_ptr(), C, sl.data_ptr(), pos.data_ptr(), back.data_ptr(),
                tf.data_ptr(), tc.data_ptr(), len(f), H, G, d, dv, C, a["scale"], a["softcap"], 0.5)
        if tensor:
            lib.lm_check(attend(*args, out.data_ptr(), H * dv + 2, _st()), "chunk_attention_prompt")
        else:
            ws = torch.empty(max(16, int(L.ao_lm_chunk_attention_workspace_bytes(len(f), G, dv, n_split))), dtype=torch.uint8, device="cuda")
            lib.lm_check(attend(*args, n_split, ws.data_ptr(), ws.numel(), out.data_ptr(), H * dv + 2, _st()), "chunk_attention")
        lib.lm_check(L.ao_lm_ring_append(kn.data_ptr(), vn.data_ptr(), c, G * d, G * dv, C, dt, sl.data_ptr(), pos.data_ptr(),
                                         ahead.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), _st()), "ring_append")
        assert float(out[:, H * dv:].abs().max()) == 0.0
        got.append(out[:, :H * dv].double().cpu())
        at += c
    assert at == h.shape[0]
    return torch.cat(got)


ATTN_SHAPES = [dict(heads=6, kv_heads=2, dim=8, vdim=12, chunk=8, rows=6, bias_max=20),
               dict(heads=2, kv_heads=2, dim=16, vdim=16, chunk=5, rows=7, bias_max=4),
               dict(heads=4, kv_heads=1, dim=32, vdim=64, chunk=16, rows=16, bias_max=12),
               dict(heads=3, kv_heads=3, dim=5, vdim=3, chunk=1, rows=2, bias_max=3),
               dict(heads=8, kv_heads=4, dim=64, vdim=48, chunk=80, rows=32, bias_max=128),
               dict(heads=2, kv_heads=1, dim=128, vdim=128, chunk=96, rows=8, bias_max=50)]


def _forms(dtype, a):
    """The forms of the attention kernel that cover a storage type and shape: fp32 arithmetic always, tensor cores for
    bf16 with head sizes in multiples of 16."""
    ok = dtype == torch.bfloat16 and a["dim"] % 16 == 0 and a["vdim"] % 16 == 0 and a["vdim"] <= 128
    return [False, True] if ok else [False]


@pytest.mark.parametrize("shape", range(len(ATTN_SHAPES)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_chunk_attention_prompt_portions_decode_and_chunk_edges(shape, dtype):
    kw = ATTN_SHAPES[shape]
    cfg = O.make_config([O.attention_layer(**kw)], width=24)
    a = cfg["layers"][0]["mixer"]["left"]
    C = a["mask"]["size"]
    w = {k: v.double() for k, v in O.random_weights(cfg, 11).items()}
    w["l0.mix.left.o"] = torch.eye(a["heads"] * a["vdim"], dtype=F64)
    T = 3 * C + 9
    h = torch.randn(T, 24, generator=torch.Generator().manual_seed(12), dtype=F64)
    ref = 0.5 * O.chunk_attention(h, w, "l0.mix.left.", a, 1e-6)
    # cuts: a portion that ends inside a chunk, single tokens over a chunk's edge, a portion over several chunks
    cuts = [max(1, C // 2), 1, 1]
    rest = T - sum(cuts)
    cuts += [rest - 4, 2, 1, 1]
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    for tensor in _forms(dtype, a):
        got = _attention_alone(a, w, h, cuts, dtype, tensor=tensor)
        assert torch.allclose(got, ref, **tol), tensor
        whole = _attention_alone(a, w, h, [T], dtype, tensor=tensor)
        assert torch.allclose(whole, ref, **tol), tensor
        assert torch.allclose(whole, got, **(dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else tol)), tensor
    # the keys of a tile spread over several CTAs (more shares than key blocks included) and merged
    for n_split in (2, 5):
        got = _attention_alone(a, w, h, cuts, dtype, n_split=n_split)
        assert torch.allclose(got, ref, **tol), n_split


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key,query", [(16, 31), (15, 16), (16, 16), (31, 32), (0, 15), (17, 30), (32, 47), (47, 48)])
def test_chunk_attention_one_dominant_key_inside_and_outside_the_chunk(dtype, key, query):
    """One key is made to match one query far better than every other key, and its value stands out.  Inside the
    query's chunk it must take nearly all the weight, in the chunk before it must not be seen at all — from a prompt
    row and from a row decoded alone."""
    kw = dict(heads=2, kv_heads=1, dim=16, vdim=16, chunk=16, rows=8, bias_max=16, scale=3.0, softcap=200.0)
    cfg = O.make_config([O.attention_layer(**kw)], width=32)
    a = cfg["layers"][0]["mixer"]["left"]
    w = {k: v.double() for k, v in O.random_weights(cfg, 13).items()}
    p = "l0.mix.left."
    eye = torch.cat([torch.eye(16, dtype=F64), torch.zeros(16, 16, dtype=F64)], 1)      # queries and keys read the first half
    w[p + "o"] = torch.eye(32, dtype=F64)
    w[p + "q"], w[p + "k"] = torch.cat([eye, eye]), eye
    w[p + "v"][:, :16] = 0.0                                                           # values read the second half
    w[p + "rel"] = torch.zeros_like(w[p + "rel"])
    w[p + "g"] = torch.zeros_like(w[p + "g"])
    T = 50
    h = torch.randn(T, 32, generator=torch.Generator().manual_seed(14), dtype=F64)
    h[key, :16] = h[query, :16]            # the same direction as the query's own key: the largest possible score
    v_key, v_own = w[p + "v"] @ h[key], w[p + "v"] @ h[query]
    ref = 0.5 * O.chunk_attention(h, w, p, a, 1e-6)
    same_chunk = key // 16 == query // 16 and key <= query
    # gate 1/2, branch scale 1/2: the far key shares the weight with the query's own key, or is not there at all
    expect = 0.25 * (0.5 * (v_key + v_own) if same_chunk else v_own)
    assert torch.allclose(ref[query, :16], expect, rtol=0, atol=1e-3)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    for cuts in ([T], [query, 1, T - query - 1], [key + 1, T - key - 1] if key + 1 < T else [T]):
        cuts = [c for c in cuts if c > 0]
        for tensor in _forms(dtype, a):
            got = _attention_alone(a, w, h, cuts, dtype, tensor=tensor)
            assert torch.allclose(got[query], ref[query], **tol), (cuts, tensor)
            assert torch.allclose(got, ref, **tol), (cuts, tensor)


def test_gelu_gated_product():
    lib, L = _lm()
    g = torch.Generator().manual_seed(15)
    for ff in (17, 64):
        gu = (torch.randn(5, 2 * ff, generator=g) * 3)
        gd, y = gu.cuda(), torch.empty(5, ff, device="cuda")
        lib.lm_check(L.ao_lm_gelu_glu(gd.data_ptr(), lib.DT_F32, 5, ff, y.data_ptr(), _st()), "gelu_glu")
        ref = O.gelu_tanh(gu.double()[:, :ff]) * gu.double()[:, ff:]
        assert torch.allclose(y.double().cpu(), ref, rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------------------------------------ the model
def _mixed():
    return O.make_config([O.recurrent_layer(24, 3, 3, ff=40), O.attention_layer(), O.recurrent_layer(20, 1, 2),
                          O.attention_layer(heads=2, kv_heads=2, dim=16, vdim=8, chunk=5, rows=7, bias_max=4, right=40, ff=0)],
                         width=32, streams=3, taps=3, loop=(1, 3, 2))


def _plain():
    """No streams, no mixer convolution, no loop, one key/value head, uncapped scores."""
    lay = O.attention_layer(heads=3, kv_heads=1, dim=8, vdim=8, chunk=6, softcap=0.0, ff=24)
    return O.make_config([lay, O.recurrent_layer(16, 2, 4, ff=24)], width=24, streams=0, taps=0)


def _ones():
    """Sizes that make things equal or one: one stream WITH weights, convolutions of one tap, a loop that runs once,
    chunks of one position, blocks of one channel, one head."""
    return O.make_config([O.attention_layer(heads=1, kv_heads=1, dim=4, vdim=4, chunk=1, rows=2, bias_max=2, right=16),
                          O.recurrent_layer(16, 16, 1), O.recurrent_layer(16, 1, 2)], width=16, streams=1, taps=1, loop=(0, 3, 1))


def _tensor():
    """Head sizes and chunks that the tensor-core attention path takes, several passes of a loop."""
    return O.make_config([O.attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, chunk=32, rows=16, bias_max=40, right=48, ff=64),
                          O.recurrent_layer(64, 2, 4)], width=64, vocab=97, streams=2, taps=4, loop=(0, 2, 3))


def _odd():
    """Nothing is a multiple of 2, 4 or 16: width, vocabulary, head sizes, recurrence widths, feed-forward, chunk."""
    return O.make_config([O.attention_layer(heads=3, kv_heads=3, dim=7, vdim=5, chunk=9, rows=5, bias_max=7, right=21, ff=25),
                          O.recurrent_layer(21, 3, 3, ff=0), O.attention_layer(heads=5, kv_heads=1, dim=3, vdim=9, chunk=11, rows=9, right=13, ff=0)],
                         width=35, vocab=53, streams=5, taps=5, loop=(1, 3, 3))


CONFIGS = {"mixed": _mixed, "plain": _plain, "ones": _ones, "tensor": _tensor, "odd": _odd}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_and_every_layer_run_against_oracle(name, dtype):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 21)
    toks = _tokens(cfg, 45, 1)
    ref, ref_layers = O.forward(cfg, w, toks, return_layers=True)
    m = _model(cfg, w, dtype)
    logits, sums = m.step_engine.layer_sums(m.states.slot_of("a"), toks)
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    assert _err(logits, ref) <= tol
    if dtype == torch.float32:
        assert sums.shape == ref_layers.shape
        for r in range(sums.shape[0]):     # small coordinates beside large ones: the bound follows the run's largest value
            scale = float(ref_layers[r].abs().max())
            assert torch.allclose(sums[r].double().cpu(), ref_layers[r], rtol=1e-4, atol=1e-5 * max(1.0, scale)), r


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_equals_token_by_token_and_portions(dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 22)
    toks = _tokens(cfg, 60, 2)
    ref = O.forward(cfg, w, toks)
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    m = _model(cfg, w, dtype)
    eng, st = m.step_engine, m.states
    for cuts in ([60], [1] * 60, [2, 2, 3, 2, 7, 1, 1, 17, 2, 23], [31, 1, 1, 1, 26]):
        got, at = [], 0
        for c in cuts:
            got.append(eng.step([(st.slot_of("r"), toks[at:at + c])], "all"))
            at += c
        st.release("r")
        assert _err(torch.cat(got), ref) <= tol, cuts


@pytest.mark.parametrize("min_rows", [1, 10 ** 9])
def test_either_attention_form_for_every_portion_and_batch(monkeypatch, min_rows):
    """The switch between the two forms of the attention kernel is a matter of speed: with the tensor-core form forced
    for every step (single decoded tokens included), and with it switched off, the logits stay the oracle's."""
    from torchao_fork_b200._models.tadolix import step as S
    monkeypatch.setattr(S, "PROMPT_MIN_ROWS", min_rows)
    cfg = _tensor()
    w = O.random_weights(cfg, 29)
    ta, tb = _tokens(cfg, 75, 9), _tokens(cfg, 40, 10)
    ra, rb = O.forward(cfg, w, ta), O.forward(cfg, w, tb)
    tol = max(_bf16_tol(cfg, w, ta), _bf16_tol(cfg, w, tb))
    m = _model(cfg, w, torch.bfloat16)
    eng, st = m.step_engine, m.states
    ga = [eng.step([(st.slot_of("a"), ta[:33])], "all")]
    both = eng.step([(st.slot_of("a"), ta[33:70]), (st.slot_of("b"), tb[:38])], "all")
    ga.append(both[:37])
    gb = [both[37:]]
    for i in range(2):
        both = eng.step([(st.slot_of("b"), tb[38 + i:39 + i]), (st.slot_of("a"), ta[70 + i:71 + i])], "all")
        gb.append(both[:1])
        ga.append(both[1:])
    ga.append(eng.step([(st.slot_of("a"), ta[72:])], "all"))
    assert _err(torch.cat(ga), ra) <= tol and _err(torch.cat(gb), rb) <= tol


def test_scan_tiles_and_pieces_cut_inside_a_step(monkeypatch):
    from torchao_fork_b200._models.tadolix import step as S
    cfg = _mixed()
    w = O.random_weights(cfg, 23)
    toks = _tokens(cfg, 70, 3)
    ref = O.forward(cfg, w, toks)
    m = _model(cfg, w)
    monkeypatch.setattr(S, "SCAN_TILE", 4)          # recurrences in three launches over 4-row tiles
    got = m.step_engine.step([(m.states.slot_of("a"), toks)], "all")
    assert _err(got, ref) <= F32_TOL
    monkeypatch.setattr(S, "MAX_STEP_TOKENS", 13)   # the step itself in pieces of 13 rows
    got = m.step_engine.step([(m.states.slot_of("b"), toks)], "all")
    assert _err(got, ref) <= F32_TOL
    both = m.step_engine.step([(m.states.slot_of("c"), toks[:40]), (m.states.slot_of("d"), toks[:9])], [[39, 3], [8]])
    assert _err(both, ref[[39, 3, 8]]) <= F32_TOL


@pytest.mark.parametrize("name", ["mixed", "plain", "tensor"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batches_of_unequal_requests_equal_each_alone_and_slots_are_reused(dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 24)
    reqs = {k: _tokens(cfg, n, 10 + i) for i, (k, n) in enumerate([("a", 37), ("b", 9), ("c", 21), ("d", 30), ("e", 5)])}
    ref = {k: O.forward(cfg, w, t) for k, t in reqs.items()}
    tol = F32_TOL if dtype == torch.float32 else max(_bf16_tol(cfg, w, t) for t in reqs.values())
    m = _model(cfg, w, dtype, slots=2)      # three live requests force the state to grow
    eng, st = m.step_engine, m.states
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    # every step: (request, tokens) pairs; requests end, their slots go to the next ones
    plan = [[("a", 11), ("b", 2)], [("a", 1), ("b", 7), ("c", 6)], [("c", 15), ("a", 1)], [("d", 30), ("a", 24)], [("e", 3)], [("e", 1)], [("e", 1)]]
    for step in plan:
        segs, names = [], []
        for k, c in step:
            segs.append((st.slot_of(k), reqs[k][at[k]:at[k] + c]))
            names.append((k, c))
            at[k] += c
        out = eng.step(segs, "all")
        r = 0
        for k, c in names:
            got[k].append(out[r:r + c])
            r += c
            if at[k] == len(reqs[k]):
                st.release(k)
    assert m.max_batch_size >= 3 and st.alloc.in_use == 0
    for k in reqs:
        assert at[k] == len(reqs[k])
        assert _err(torch.cat(got[k]), ref[k]) <= tol, k


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_wraps_the_ring_many_times_and_remembers_far_tokens(dtype):
    cfg = _mixed()
    w = O.random_weights(cfg, 25)
    toks = _tokens(cfg, 150, 4)
    ref = O.forward(cfg, w, toks)
    # the recurrences carry the first token to the end: another first token moves the last logits
    other = O.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert _err(other[-1:], ref[-1:]) > 1e-3
    m = _model(cfg, w, dtype)
    eng, st = m.step_engine, m.states
    got = [eng.step([(st.slot_of("r"), toks[:20])], "all")] + [eng.step([(st.slot_of("r"), [t])], "all") for t in toks[20:]]
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    assert _err(torch.cat(got), ref) <= tol


@pytest.mark.parametrize("batch", [1, 2])
def test_greedy_generation_through_generator_and_graph(batch):
    from torchao_fork_b200._models.llama.generate import Generator
    cfg = _mixed()
    w = O.random_weights(cfg, 26)
    prompt = _tokens(cfg, 13, 5)
    want = O.greedy(cfg, w, prompt, 12)
    for use_graph in (False, True):
        m = _model(cfg, w, torch.float32, slots=batch)
        gen = Generator(m, batch, 64, temperature=0.0, top_k=None, use_graph=use_graph)
        for _ in range(2):      # the second call restarts the slots at position 0
            seq = gen.generate(torch.tensor(prompt), 12)
            assert seq.shape == (batch, 25)
            for b in range(batch):
                assert seq[b, 13:].tolist() == want, (use_graph, b)


def test_sampling_with_temperature_runs_through_the_framework_sampler():
    from torchao_fork_b200._models.llama.generate import Generator
    cfg = _plain()
    m = _model(cfg, O.random_weights(cfg, 27), torch.bfloat16, slots=1)
    gen = Generator(m, 1, 40, temperature=0.8, top_k=5, use_graph=True)
    seq = gen.generate(torch.tensor(_tokens(cfg, 6, 6)), 10)
    assert seq.shape == (1, 16) and int(seq.min()) >= 0 and int(seq.max()) < cfg["vocab"]


def test_named_configuration_through_the_registry():
    from torchao_fork_b200._models import registry
    m = registry.random_init("Tadolix-test", "cuda", torch.bfloat16)
    m.setup_caches(1, 64)
    out = m(torch.randint(0, 512, (1, 20), device="cuda"))
    assert out.shape == (1, 1, 512) and bool(torch.isfinite(out).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_on_a_checkpoint_folder(tmp_path, dtype):
    cfg = _mixed()
    w = O.random_weights(cfg, 28)
    folder, out = str(tmp_path / "model"), str(tmp_path / "out")
    O.write_checkpoint(folder, cfg, w)
    a, b = _tokens(cfg, 29, 7), _tokens(cfg, 12, 8)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[17:19], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[19:], "want": [9]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[:11], "want": [10]}], "end": []},
             {"step": 4, "entries": [{"id": "b", "tokens": b[11:], "want": [0]}], "end": ["b"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                        "--max-tokens", "64", "--slots", "1"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    ra, rb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    tol = F32_TOL if dtype == "float32" else max(_bf16_tol(cfg, w, a), _bf16_tol(cfg, w, b))
    V = cfg["vocab"]
    rd = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, V).copy())
    assert _err(rd(0), ra[[0, 16]]) <= tol and _err(rd(2), ra[[28]]) <= tol
    assert _err(rd(3), rb[[10]]) <= tol and _err(rd(4), rb[[11]]) <= tol
