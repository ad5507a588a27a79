"""Bitipel on the GPU against the float64 oracle (tests/bitipel_oracle.py): every mechanism's kernel alone, then the model
through the framework's step function, state manager, decode engine and Generator.  Configurations and weights are
made here; float32 runs are held to a tight bound (only summation order differs), bfloat16 runs to the rounding noise
of bf16 products."""
import ctypes
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import bitipel_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 2e-4


def _bf16_tol(cfg, w, toks):
    """A bfloat16 run may be 3 times as far from the exact logits as bfloat16 rounding alone moves them (measured by the
    oracle rounding where such a run rounds), for this model and input."""
    return 3.0 * O.rounding_noise(cfg, w, toks, _err)


def _lm():
    from torchao_fork_b200 import _lib
    return _lib, _lib.lm()


def _model(cfg, w, dtype=torch.float32, slots=2, seq=96):
    from torchao_fork_b200._models.bitipel import Bitipel, BitipelArgs
    m = Bitipel(BitipelArgs.from_dict(cfg), w, "cuda", dtype).eval()
    m.setup_caches(slots, seq)
    return m


def _err(got, ref):
    """Root mean square of the difference (mean over the vocabulary taken off), relative to the reference's spread."""
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def _tokens(cfg, n, seed=0):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _st():
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_kernel_rows_state_and_sequence_starts(dtype):
    lib, L = _lm()
    W, dt = 70, (lib.DT_F32 if dtype == torch.float32 else lib.DT_BF16)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(6, W, generator=g)
    mu = torch.rand(W, generator=g).to(dtype)
    state = torch.randn(3, W, generator=g)
    # rows: slot 2 continues at position 5 (reads state), 6; slot 0 starts at position 0 (zeros), 1, 2; slot 1 decodes at 9
    slot = torch.tensor([2, 2, 0, 0, 0, 1], dtype=torch.int32)
    pos = torch.tensor([5, 6, 0, 1, 2, 9], dtype=torch.int32)
    h = torch.empty(6, W, dtype=dtype, device="cuda")
    xd, mud, std, sld, pd = x.cuda(), mu.cuda(), state.cuda(), slot.cuda(), pos.cuda()   # kept alive until the kernel has run
    lib.lm_check(L.ao_lm_token_shift(xd.data_ptr(), mud.data_ptr(), dt, std.data_ptr(), sld.data_ptr(),
                                     pd.data_ptr(), 6, W, h.data_ptr(), _st()), "token_shift")
    xf, muf = x.double(), mu.double()
    ref = torch.cat([O.token_shift(xf[0:2], muf, state[2].double()), O.token_shift(xf[2:5], muf, torch.zeros(W, dtype=O.F64)),
                     O.token_shift(xf[5:6], muf, state[1].double())])
    assert torch.allclose(h.double().cpu(), ref, rtol=1e-6 if dtype == torch.float32 else 1e-2, atol=1e-6 if dtype == torch.float32 else 2e-2)


def test_residual_norm_kernel_with_state_average_and_copy():
    lib, L = _lm()
    n, W, ns = 5, 50, 3
    g = torch.Generator().manual_seed(2)
    x = torch.randn(n, W, generator=g)
    y = (torch.randn(n, W, generator=g) * 3).to(torch.bfloat16)
    gw = torch.tensor([1.3], dtype=torch.bfloat16)
    coef = torch.randn(ns + 1, generator=g).to(torch.bfloat16)
    streams = torch.randn(ns + 1, n, W, generator=g).cuda()
    slot = torch.tensor([1, 1, 1, 0, 0], dtype=torch.int32).cuda()
    state = torch.zeros(2, W).cuda()
    avg = torch.empty(n, W).cuda()
    cast = torch.empty(n, W, dtype=torch.bfloat16).cuda()
    xd, yd, gd, cd = x.cuda(), y.cuda(), gw.cuda(), coef.cuda()
    lib.lm_check(L.ao_lm_residual_norm(xd.data_ptr(), yd.data_ptr(), lib.DT_BF16, gd.data_ptr(), lib.DT_BF16, 0.6, 1e-5, n, W,
                                       streams[ns].data_ptr(), state.data_ptr(), slot.data_ptr(), streams.data_ptr(), ns, n * W,
                                       cd.data_ptr(), avg.data_ptr(), cast.data_ptr(), _st()), "residual_norm")
    xo = x.double() + 0.6 * O.scalar_norm(y.double(), gw.double(), 1e-5)
    assert torch.allclose(streams[ns].double().cpu(), xo, rtol=1e-5, atol=1e-5)
    ref_avg = O.depth_average([streams[j].double().cpu() for j in range(ns)] + [xo], coef.double())
    assert torch.allclose(avg.double().cpu(), ref_avg, rtol=1e-5, atol=1e-5)
    assert torch.allclose(cast.double().cpu(), ref_avg, rtol=1e-2, atol=1e-2)
    # the last row of each sequence in the batch leaves the layer's INPUT row behind
    assert torch.equal(state[1].cpu(), x[2]) and torch.equal(state[0].cpu(), x[4])


@pytest.mark.parametrize("H,dn,dr,R,rot", [(3, 8, 6, 40, 6), (4, 16, 8, 64, 4), (1, 4, 2, 33, 2)])
def test_latent_prep_kernel_norm_rotation_cache_rows(H, dn, dr, R, rot):
    lib, L = _lm()
    n, S, base, eps = 4, 3000, 50000.0, 1e-5
    g = torch.Generator().manual_seed(3)
    ld = H * (dn + dr) + R + dr + H
    proj = torch.randn(n, ld, generator=g)
    cn = (1 + 0.2 * torch.randn(R, generator=g))
    slot = torch.tensor([1, 1, 0, 1], dtype=torch.int32)
    pos = torch.tensor([0, 1, 2999, 2047], dtype=torch.int32)      # far positions: the angle must be exact in fp32
    inv = torch.tensor([base ** (-2.0 * j / rot) for j in range(rot // 2)], dtype=torch.float64).float().cuda()
    c = torch.zeros(2, S, R).cuda()
    kr = torch.zeros(2, S, dr).cuda()
    qn = torch.empty(H, n, dn).cuda()
    qr = torch.empty(n, H, dr).cuda()
    gate = torch.empty(n, H).cuda()
    pjd, cnd, sld, pd = proj.cuda(), cn.cuda(), slot.cuda(), pos.cuda()
    lib.lm_check(L.ao_lm_latent_prep(pjd.data_ptr(), lib.DT_F32, ld, n, H, dn, dr, R, 0, H * (dn + dr), H * (dn + dr) + R + dr,
                                     cnd.data_ptr(), eps, rot, inv.data_ptr(), sld.data_ptr(), pd.data_ptr(),
                                     c.data_ptr(), kr.data_ptr(), S, qn.data_ptr(), qr.data_ptr(), gate.data_ptr(), _st()), "latent_prep")
    p = proj.double()
    q = p[:, : H * (dn + dr)].view(n, H, dn + dr)
    assert torch.allclose(qn.double().cpu(), q[..., :dn].transpose(0, 1), atol=1e-7)
    assert torch.allclose(qr.double().cpu(), O.rotate_pairs(q[..., dn:], pos, base, rot), atol=2e-4, rtol=1e-4)
    assert torch.allclose(gate.double().cpu(), torch.sigmoid(p[:, -H:]), atol=1e-6)
    lat = p[:, H * (dn + dr):H * (dn + dr) + R + dr]
    for t in range(n):
        assert torch.allclose(c[slot[t], pos[t]].double().cpu(), O.vector_norm(lat[t, :R], cn.double(), eps), atol=1e-5, rtol=1e-5)
        assert torch.allclose(kr[slot[t], pos[t]].double().cpu(), O.rotate_pairs(lat[t:t + 1, R:], pos[t:t + 1], base, rot)[0],
                              atol=2e-4, rtol=1e-4)
    assert int((c.abs().sum(-1) > 0).sum()) == n          # no other row was touched


def _attention_case(H, R, dr, segs, S, dtype, n_split, far=None, seed=4):
    """segs: [(slot, first position, count)].  Runs the kernel on random queries and cached rows; returns (got, reference)."""
    lib, L = _lm()
    dt = lib.DT_F32 if dtype == torch.float32 else lib.DT_BF16
    g = torch.Generator().manual_seed(seed)
    n_slots = max(s for s, _, _ in segs) + 1
    c = torch.randn(n_slots, S, R, generator=g).to(dtype)
    kr = torch.randn(n_slots, S, dr, generator=g).to(dtype)
    slot = torch.cat([torch.full((k,), s) for s, _, k in segs]).int()
    pos = torch.cat([torch.arange(p, p + k) for _, p, k in segs]).int()
    n = len(slot)
    qa = torch.randn(H, n, R, generator=g)
    qr = torch.randn(n, H, dr, generator=g)
    if far is not None:       # (row, head, key): that key's latent is aligned with the row's query so that its score stands out
        t, h, key = far
        c[slot[t], key] = (qa[h, t] / qa[h, t].norm() * 6.0).to(dtype)
    sink = torch.randn(H, generator=g).to(dtype)
    gate = torch.rand(n, H, generator=g)
    scale = 1.0 / math.sqrt(R + dr) * 2.0
    tt = ctypes.c_int()
    lib.lm_check(L.ao_lm_latent_attention_plan(dt, H, R, dr, ctypes.byref(tt)), "plan")
    first, count = [], []
    at = 0
    for _, _, k in segs:
        for f in range(at, at + k, tt.value):
            first.append(f)
            count.append(min(tt.value, at + k - f))
        at += k
    tf, tc = torch.tensor(first).int().cuda(), torch.tensor(count).int().cuda()
    ws = torch.zeros(max(16, int(L.ao_lm_latent_attention_workspace_bytes(n, H, R, n_split))), dtype=torch.uint8, device="cuda")
    out = torch.full((n, H, R), float("nan"), dtype=dtype, device="cuda")
    cd, krd, qad, qrd, sld, pd, skd, gd = c.cuda(), kr.cuda(), qa.cuda(), qr.cuda(), slot.cuda(), pos.cuda(), sink.cuda(), gate.cuda()
    lib.lm_check(L.ao_lm_latent_attention(qad.data_ptr(), qrd.data_ptr(), cd.data_ptr(), krd.data_ptr(), dt, S,
                                          sld.data_ptr(), pd.data_ptr(), tf.data_ptr(), tc.data_ptr(), len(first), n, H, R, dr,
                                          scale, skd.data_ptr(), gd.data_ptr(), int(pos.max()), n_split, ws.data_ptr(),
                                          ws.numel(), out.data_ptr(), _st()), "latent_attention")
    ref = torch.empty(n, H, R, dtype=O.F64)
    for t in range(n):
        ks = c[slot[t], : pos[t] + 1].double()
        s = (torch.einsum("hr,sr->hs", qa[:, t].double(), ks) + torch.einsum("hd,sd->hs", qr[t].double(), kr[slot[t], : pos[t] + 1].double())) * scale
        p = O.sink_softmax(s, sink.double().view(H, 1))
        ref[t] = (p @ ks) * gate[t].double().view(H, 1)
    return out.double().cpu(), ref


@pytest.mark.parametrize("H,R,dr", [(4, 64, 8), (3, 40, 6), (9, 33, 2), (2, 130, 16), (1, 16, 4), (4, 64, 16), (3, 128, 32), (20, 192, 16), (16, 512, 64)])
@pytest.mark.parametrize("n_split", [1, 3])
def test_latent_attention_kernel_prompt_decode_and_mixed_rows(H, R, dr, n_split):
    # a prompt portion that starts in the middle of a key tile, a decoded token far in, the first tokens of a sequence
    segs = [(0, 29, 9), (1, 150, 1), (2, 0, 3)]
    got, ref = _attention_case(H, R, dr, segs, 160, torch.float32, n_split)
    assert torch.allclose(got, ref, rtol=2e-5, atol=2e-5)
    got, ref = _attention_case(H, R, dr, segs, 160, torch.bfloat16, n_split)
    assert torch.allclose(got, ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("key", [0, 31, 32, 33, 63, 64, 255, 256, 699])
def test_latent_attention_kernel_finds_one_far_key(key):
    """One key among 700 carries almost all the weight: at tile borders, at split borders, first and last."""
    for n_split in (1, 4, 7):
        got, ref = _attention_case(2, 48, 4, [(0, 699, 1)], 704, torch.float32, n_split, far=(0, 1, key))
        assert torch.allclose(got, ref, rtol=2e-5, atol=2e-5)
        assert float(ref[0, 1].abs().max()) > 0.3          # the far key did dominate that head
        got, ref = _attention_case(5, 64, 16, [(0, 699, 1)], 704, torch.bfloat16, n_split, far=(0, 3, key))   # tensor-core path
        assert torch.allclose(got, ref, rtol=1e-2, atol=1e-2) and float(ref[0, 3].abs().max()) > 0.3
    # the same key seen from inside a prompt portion, just visible and not yet visible
    if key >= 2:
        got, ref = _attention_case(2, 48, 4, [(0, key - 2, 5)], 704, torch.float32, 1, far=(2, 0, key))
        assert torch.allclose(got, ref, rtol=2e-5, atol=2e-5)


def _expanded_case(H, dn, dr, dv, segs, S, far=None, seed=5):
    """The prompt-portion kernel on random queries, per-head keys / values and cached rotated key parts.
    segs: [(slot, first position, count)]; every sequence's keys 0 .. its last position lie one after the other."""
    lib, L = _lm()
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    n_slots = max(s for s, _, _ in segs) + 1
    slot = torch.cat([torch.full((k,), s) for s, _, k in segs]).int()
    pos = torch.cat([torch.arange(p, p + k) for _, p, k in segs]).int()
    n = len(slot)
    qn = torch.randn(H, n, dn, generator=g).to(bf)
    qr = torch.randn(n, H, dr, generator=g)
    kr = torch.randn(n_slots, S, dr, generator=g).to(bf)
    rows, row0 = 0, {}
    for s, p, k in segs:
        row0[s] = rows
        rows += p + k
    kx = torch.randn(rows, H, dn, generator=g).to(bf)
    vx = torch.randn(rows, H, dv, generator=g).to(bf)
    if far is not None:       # (row, head, key): that key is aligned with the row's query so that its score stands out
        t, h, key = far
        kx[row0[int(slot[t])] + key, h] = (qn[h, t].float() / qn[h, t].float().norm() * 8.0).to(bf)
    sink = torch.randn(H, generator=g).to(bf)
    gate = 0.5 + 0.5 * torch.rand(n, H, generator=g)
    scale = 1.0 / math.sqrt(dn + dr) * 2.0
    tt = ctypes.c_int()
    lib.lm_check(L.ao_lm_latent_attention_expanded_plan(lib.DT_BF16, dn, dr, dv, ctypes.byref(tt)), "plan")
    assert tt.value > 0
    first, count, kvrow = [], [], []
    at = 0
    for s, _, k in segs:
        for f in range(at, at + k, tt.value):
            first.append(f)
            count.append(min(tt.value, at + k - f))
            kvrow.append(row0[s])
        at += k
    dev = lambda t: t.cuda()
    tf, tc, tr = dev(torch.tensor(first).int()), dev(torch.tensor(count).int()), dev(torch.tensor(kvrow).int())
    out = torch.full((n, H, dv), float("nan"), dtype=bf, device="cuda")
    d = [dev(t) for t in (qn, qr, kx, vx, kr, slot, pos, sink, gate)]
    lib.lm_check(L.ao_lm_latent_attention_expanded(
        d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), d[4].data_ptr(), lib.DT_BF16, S, d[5].data_ptr(),
        d[6].data_ptr(), tf.data_ptr(), tc.data_ptr(), tr.data_ptr(), len(first), n, H, dn, dr, dv, scale, d[7].data_ptr(),
        d[8].data_ptr(), out.data_ptr(), _st()), "latent_attention_expanded")
    ref = torch.empty(n, H, dv, dtype=O.F64)
    for t in range(n):
        sl, last = int(slot[t]), int(pos[t]) + 1
        k = kx[row0[sl]: row0[sl] + last].double()
        sc = (torch.einsum("hd,shd->hs", qn[:, t].double(), k) + torch.einsum("hd,sd->hs", qr[t].double(), kr[sl, :last].double())) * scale
        p = O.sink_softmax(sc, sink.double().view(H, 1))
        ref[t] = torch.einsum("hs,shd->hd", p, vx[row0[sl]: row0[sl] + last].double()) * gate[t].double().view(H, 1)
    return out.double().cpu(), ref


@pytest.mark.parametrize("H,dn,dr,dv", [(3, 16, 16, 32), (2, 32, 0, 64), (5, 48, 32, 112), (1, 16, 32, 16), (4, 128, 64, 128)])
def test_expanded_attention_kernel_portions_tiles_and_first_tokens(H, dn, dr, dv):
    # a portion that starts inside a key tile and spans three row tiles, one row far in, the first tokens, a full tile
    segs = [(0, 29, 140), (1, 150, 1), (2, 0, 3), (3, 64, 64)]
    got, ref = _expanded_case(H, dn, dr, dv, segs, 176)
    assert torch.allclose(got, ref, rtol=1e-2, atol=1e-2)
    assert float((got - ref).abs().max()) < 1.2e-2 and float((got - ref).pow(2).mean().sqrt()) < 2e-3   # bf16 output rounding only


@pytest.mark.parametrize("key", [0, 1, 62, 63, 64, 65, 127, 128, 300])
def test_expanded_attention_kernel_finds_one_far_key_and_respects_the_mask(key):
    """One key carries almost all the weight of one row: seen from rows before it (masked), at it and after it."""
    for first in (max(0, key - 2), max(0, key - 63), max(0, key - 64)):
        count = 70
        t = key - first           # the row AT the key
        for row in (t, min(count - 1, t + 1), count - 1):
            got, ref = _expanded_case(2, 16, 16, 32, [(0, first, count)], first + count, far=(row, 1, key))
            assert torch.allclose(got, ref, rtol=1e-2, atol=1e-2), (first, row)
            assert float(ref[row, 1].abs().max()) > 0.2


@pytest.mark.parametrize("E,top,W", [(5, 2, 70), (1, 1, 64), (40, 6, 96), (8, 8, 33)])
def test_router_kernel_softmax_over_all_then_top(E, top, W):
    lib, L = _lm()
    g = torch.Generator().manual_seed(6)
    h = torch.randn(7, W, generator=g).to(torch.bfloat16)
    wr = (torch.randn(E, W, generator=g) * 0.5).to(torch.bfloat16)
    idx = torch.empty(7, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(7, top, device="cuda")
    hd, wrd = h.cuda(), wr.cuda()
    lib.lm_check(L.ao_lm_router_topk(hd.data_ptr(), wrd.data_ptr(), lib.DT_BF16, 7, W, E, top, idx.data_ptr(), wt.data_ptr(), _st()), "router")
    rw, ri = O.route(h.double(), wr, top)
    assert torch.equal(idx.cpu().long(), ri)
    assert torch.allclose(wt.double().cpu(), rw, rtol=1e-5, atol=1e-7)
    assert top == E or float(wt.sum(-1).max()) < 1.0       # scores of the chosen, not renormalised
    # the same choice from logits that a GEMM made (what prompt portions use); 19 tokens: more than one CTA of warps
    h2 = torch.randn(19, W, generator=g).to(torch.bfloat16)
    z = (h2.double() @ wr.double().T).float().cuda()
    idx2 = torch.empty(19, top, dtype=torch.int32, device="cuda")
    wt2 = torch.empty(19, top, device="cuda")
    lib.lm_check(L.ao_lm_router_topk_logits(z.data_ptr(), 19, E, top, idx2.data_ptr(), wt2.data_ptr(), _st()), "router_logits")
    rw, ri = O.route(h2.double(), wr, top)
    assert torch.equal(idx2.cpu().long(), ri) and torch.allclose(wt2.double().cpu(), rw, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_expert_kernels_and_sorted_path_against_oracle(dtype):
    """The mixture through the model's two paths (index-driven kernels for few rows, sorted rows around GEMMs for many)."""
    cfg = O.random_config(width=72, experts=5, top=2, ff=40, shared_ff=24, limit=0.8, shared_limit=1.1, n_layers=1, share=(None,))
    w = O.random_weights(cfg, seed=7)
    m = _model(cfg, w, dtype)
    eng, lay, f = m.step_engine, m.layers[0], m.config.layers[0].mlp
    g = torch.Generator().manual_seed(8)
    for n, gemv in ((3, True), (3, False), (41, False)):
        x = (torch.randn(n, 72, generator=g) * 1.5).to(dtype)
        ffo = torch.empty(n, 72, device="cuda")
        xd = x.cuda()
        eng._experts(lay, f, xd, ffo, n, gemv, _st())
        ref = O.mixture(x.double(), w, "l0.mlp.", cfg["layers"][0]["mlp"])
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        assert torch.allclose(ffo.double().cpu(), ref, rtol=tol, atol=tol * float(ref.abs().max()))
    # the clip matters in this test: some pre-activations exceed the limits
    pre = x.double() @ w["l0.mlp.e0.gate"].double().T
    assert float(pre.max()) > 0.8


@pytest.mark.parametrize("ff", [24, 17, 128])
def test_clipped_glu_activation_kernel_vector_and_scalar_rows(ff):
    """g = min(a, limit), u = clamp(b, +-limit), y = g sigmoid(1.702 g) (u + 1) on rows [a | b]; rows of 8k numbers take the
    16-byte path, others the scalar one."""
    lib, L = _lm()
    g = torch.Generator().manual_seed(9)
    gu = (torch.randn(11, 2 * ff, generator=g) * 2.0).to(torch.bfloat16)
    y = torch.empty(11, ff, dtype=torch.bfloat16, device="cuda")
    gud = gu.cuda()
    lib.lm_check(L.ao_lm_glu_act(gud.data_ptr(), lib.DT_BF16, 11, ff, 1.25, 1.702, y.data_ptr(), _st()), "glu_act")
    a, b = gu[:, :ff].double().clamp(max=1.25), gu[:, ff:].double().clamp(-1.25, 1.25)
    ref = a * torch.sigmoid(1.702 * a) * (b + 1.0)
    assert torch.allclose(y.double().cpu(), ref, rtol=1e-2, atol=1e-2)
    assert float(gu[:, :ff].max()) > 1.25 and float(gu[:, ff:].min()) < -1.25      # both clips were active


def test_argmax_kernel_first_of_ties():
    lib, L = _lm()
    lg = torch.randn(3, 1000)
    lg[1, 17] = lg[1, 900] = 50.0
    out = torch.empty(3, dtype=torch.int64, device="cuda")
    ld = lg.cuda()
    lib.lm_check(L.ao_lm_argmax(ld.data_ptr(), 1000, 3, 1000, out.data_ptr(), _st()), "argmax")
    assert out.cpu().tolist() == [int(lg[0].argmax()), 17, int(lg[2].argmax())]


# ------------------------------------------------------------------------------------------------ the model
CONFIGS = {
    # borrowing layers, a layer without feed-forward, odd head count and latent size
    "mixed": dict(width=64, vocab=97, heads=3, dim=8, rot_dim=6, vdim=10, kv_rank=40, n_layers=4, share=(None, 0, None, 2),
                  experts=5, top=2, ff=24, shared_ff=20, no_mlp=(2,)),
    # sizes that other models make equal or one are all different / not one here; one expert of one, many heads
    "wide": dict(width=96, vocab=131, heads=9, dim=4, rot_dim=2, vdim=7, kv_rank=33, n_layers=2, share=(None, None),
                 experts=1, top=1, ff=17, shared_ff=9, mult=1.3, eps=1e-3, base=123.0),
    # latent size a multiple of 64 and rotated size a multiple of 16: in bfloat16 the attention runs on the tensor cores
    "tensor": dict(width=64, vocab=89, heads=5, dim=8, rot_dim=16, vdim=12, kv_rank=64, n_layers=3, share=(None, 0, None),
                   experts=4, top=2, ff=16, shared_ff=16),
    # head sizes that the prompt-portion (expanded) attention kernel covers in bfloat16; latent size that keeps decoding
    # on the fp32 path: a step of 32 or more tokens per sequence and a smaller one take different kernels
    "expanded": dict(width=64, vocab=101, heads=3, dim=16, rot_dim=16, vdim=32, kv_rank=40, n_layers=3, share=(None, 0, None),
                     experts=6, top=2, ff=24, shared_ff=16),
    "single": dict(width=32, vocab=50, heads=1, dim=16, rot_dim=8, vdim=32, kv_rank=16, n_layers=3, share=(None, 0, 0),
                   experts=7, top=7, ff=8, shared_ff=8),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_and_every_layer_against_oracle(name, dtype):
    cfg = O.random_config(**CONFIGS[name])
    w = O.random_weights(cfg, seed=11)
    toks = _tokens(cfg, 45)
    ref, _ = O.forward(cfg, w, toks, return_layers=True)
    m = _model(cfg, w, dtype)
    got = m.step_engine.step([(m.states.slot_of("a"), toks)], "all")
    assert _err(got, ref) < (F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks))


def test_layer_results_against_oracle_layer_by_layer():
    """The stream after every layer (after the depth average), read from the step's own buffers."""
    cfg = O.random_config(**CONFIGS["mixed"])
    w = O.random_weights(cfg, seed=12)
    toks = _tokens(cfg, 20, 1)
    _, layers = O.forward(cfg, w, toks, return_layers=True)
    for upto in range(1, 5):
        sub = dict(cfg, layers=cfg["layers"][:upto])
        ws = {k: v for k, v in w.items() if not k.startswith("l") or int(k[1:k.index(".")]) < upto}
        m = _model(sub, ws, torch.float32)
        eng = m.step_engine
        st = m.states
        slot = st.slot_of("a")
        p0 = st.extend(slot, len(toks))
        x = eng._run(np.asarray(toks, np.int64), np.full(len(toks), slot, np.int32), np.arange(p0, p0 + len(toks), dtype=np.int32))
        assert torch.allclose(x.double().cpu(), layers[upto - 1], rtol=1e-4, atol=1e-4), upto


@pytest.mark.parametrize("name", ["mixed", "tensor", "expanded"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_equals_token_by_token_and_portions(dtype, name):
    _check_portions(dtype, name)


def _check_portions(dtype, name):
    cfg = O.random_config(**CONFIGS[name])
    w = O.random_weights(cfg, seed=13)
    toks = _tokens(cfg, 70, 2)
    ref = O.forward(cfg, w, toks)
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    m = _model(cfg, w, dtype)
    eng, st = m.step_engine, m.states
    for cuts in ([1] * 70, [2] * 35, [33, 2, 2, 31, 2], [64, 3, 3], [5, 1, 1, 40, 1, 22], [17, 18, 35]):
        slot = st.slot_of("r")
        outs, at = [], 0
        for k in cuts:
            outs.append(eng.step([(slot, toks[at:at + k])], "all"))
            at += k
        st.release("r")
        assert _err(torch.cat(outs), ref) < tol, cuts


def test_long_piece_is_cut_inside_the_step(monkeypatch):
    from torchao_fork_b200._models.bitipel import step as S
    cfg = O.random_config(**CONFIGS["wide"])
    w = O.random_weights(cfg, seed=14)
    toks = _tokens(cfg, 50, 3)
    ref = O.forward(cfg, w, toks)
    m = _model(cfg, w, torch.float32)
    monkeypatch.setattr(S, "MAX_STEP_TOKENS", 16)
    got = m.step_engine.step([(m.states.slot_of("a"), toks)], [[0, 15, 16, 17, 31, 32, 49]])
    assert _err(got, ref[[0, 15, 16, 17, 31, 32, 49]]) < F32_TOL


@pytest.mark.parametrize("name", ["mixed", "tensor", "expanded"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batches_of_unequal_requests_equal_each_alone_and_slots_are_reused(dtype, name):
    _check_batches(dtype, name)


def test_expanded_attention_for_every_portion_and_batch(monkeypatch):
    """With the threshold taken down, portions of two tokens and every row of a mixed batch (a sequence that brings one
    token beside longer ones, a reused slot) attend through the prompt-portion kernel."""
    from torchao_fork_b200._models.bitipel import step as S
    monkeypatch.setattr(S, "EXPAND_MIN_TOKENS", 2)
    _check_portions(torch.bfloat16, "expanded")
    monkeypatch.setattr(S, "EXPAND_MIN_TOKENS", 1)
    _check_batches(torch.bfloat16, "expanded")


def _check_batches(dtype, name):
    cfg = O.random_config(**CONFIGS[name])
    w = O.random_weights(cfg, seed=15)
    reqs = {"a": _tokens(cfg, 37, 4), "b": _tokens(cfg, 5, 5), "c": _tokens(cfg, 21, 6), "d": _tokens(cfg, 30, 7)}
    ref = {k: O.forward(cfg, w, v) for k, v in reqs.items()}
    tol = F32_TOL if dtype == torch.float32 else max(_bf16_tol(cfg, w, v) for v in reqs.values())
    m = _model(cfg, w, dtype, slots=2)          # fewer slots than requests: the state grows, and freed slots come back
    eng, st = m.step_engine, m.states
    # step 1: a's first 20 tokens + all of b + c's first token;  step 2: a decodes one, c continues with 19;  b ends
    l1 = eng.step([(st.slot_of("a"), reqs["a"][:20]), (st.slot_of("b"), reqs["b"]), (st.slot_of("c"), reqs["c"][:1])], "all")
    assert _err(l1[:20], ref["a"][:20]) < tol and _err(l1[20:25], ref["b"]) < tol and _err(l1[25:], ref["c"][:1]) < tol
    b_slot = st.slot_of("b")
    st.release("b")
    assert st.slot_of("d") == b_slot          # d inherits b's slot with b's rows still in it
    l2 = eng.step([(st.slot_of("a"), reqs["a"][20:21]), (st.slot_of("c"), reqs["c"][1:20]), (st.slot_of("d"), reqs["d"][:7])], "all")
    assert _err(l2[:1], ref["a"][20:21]) < tol and _err(l2[1:20], ref["c"][1:20]) < tol and _err(l2[20:], ref["d"][:7]) < tol
    l3 = eng.step([(st.slot_of("d"), reqs["d"][7:]), (st.slot_of("a"), reqs["a"][21:]), (st.slot_of("c"), reqs["c"][20:])], "last")
    assert _err(l3, torch.stack([ref["d"][-1], ref["a"][-1], ref["c"][-1]])) < tol


def _uneven_config():
    """Every layer with sizes and constants of its own: head counts and sizes, latent sizes, partial rotation with its own
    base, scales, expert counts / sizes / limits, with and without a shared expert, one layer without feed-forward,
    borrowing layers whose heads differ from the lender's."""
    cfg = O.random_config(width=96, vocab=113, heads=4, dim=16, rot_dim=16, vdim=32, kv_rank=64, n_layers=5,
                          share=(None, 0, None, None, 3), experts=6, top=2, ff=24, shared_ff=16, no_mlp=(3,))
    L = cfg["layers"]
    L[1]["mixer"].update(heads=6, dim=8, vdim=48, scale=0.27)
    L[1]["mlp"] = {"expert": {"ff": 8, "limit": 2.0}, "kind": "moe", "router": {"experts": 9, "top": 4},
                   "shared": {"ff": 40, "limit": 3.0}}
    L[2]["mixer"].update(heads=2, dim=32, vdim=16, kv_rank=40, rot_dim=8, scale=0.31, rot={"base": 777.0, "dims": 4})
    L[2]["mlp"] = {"expert": {"ff": 16, "limit": 0.8}, "kind": "moe", "router": {"experts": 3, "top": 3}}
    L[3]["mixer"].update(heads=1, dim=16, vdim=64, kv_rank=128, rot_dim=32, scale=0.2, rot={"base": 50.0, "dims": 32})
    L[4]["mixer"].update(heads=3, dim=32, vdim=16, kv_rank=128, rot_dim=32, scale=0.15, rot={"base": 50.0, "dims": 32})
    return cfg


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_of_unequal_sizes_whole_portions_and_decoding(dtype):
    cfg = _uneven_config()
    w = O.random_weights(cfg, seed=21)
    toks = _tokens(cfg, 90, 9)
    ref = O.forward(cfg, w, toks)
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    m = _model(cfg, w, dtype)
    eng, st = m.step_engine, m.states
    for cuts in ([90], [70] + [1] * 20, [40, 2, 33, 3, 12]):
        slot = st.slot_of("r")
        outs, at = [], 0
        for k in cuts:
            outs.append(eng.step([(slot, toks[at:at + k])], "all"))
            at += k
        st.release("r")
        assert _err(torch.cat(outs), ref) < tol, cuts


def test_rotation_and_keys_far_away_in_the_model():
    """A sequence of several hundred tokens through portions and single tokens: positions far from zero, keys far back."""
    cfg = O.random_config(width=48, vocab=61, heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=24, n_layers=2, share=(None, 0),
                          experts=3, top=1, ff=16, shared_ff=16, base=100.0)
    w = O.random_weights(cfg, seed=16)
    toks = _tokens(cfg, 400, 8)
    ref = O.forward(cfg, w, toks)
    m = _model(cfg, w, torch.float32, seq=400)
    eng, slot = m.step_engine, m.states.slot_of("a")
    got = [eng.step([(slot, toks[:350])], [[0, 1, 31, 32, 33, 349]])]
    got += [eng.step([(slot, toks[i:i + 1])], "last") for i in range(350, 400)]
    assert _err(torch.cat(got), torch.cat([ref[[0, 1, 31, 32, 33, 349]], ref[350:]])) < F32_TOL


# ------------------------------------------------------------------------------------------------ entry points
@pytest.mark.parametrize("batch", [1, 2])
def test_greedy_generation_through_generator_and_graph(batch):
    from torchao_fork_b200._models.llama.generate import Generator
    cfg = O.random_config(**CONFIGS["mixed"])
    w = O.random_weights(cfg, seed=17)
    prompt = _tokens(cfg, 9, 9)
    want = O.greedy(cfg, w, prompt, 40)
    m = _model(cfg, w, torch.float32, slots=batch, seq=64)
    gen = Generator(m, batch, 64, temperature=0.0, top_k=None)
    assert gen.engine.graph is not None
    out = gen.generate(torch.tensor(prompt), 40)
    for b in range(batch):
        assert out[b].tolist() == want
    # a second prompt on the same generator: slots and graph are reused
    prompt2 = _tokens(cfg, 4, 10)
    assert gen.generate(torch.tensor(prompt2), 12)[0].tolist() == O.greedy(cfg, w, prompt2, 12)


def test_sampling_with_temperature_runs_through_the_framework_sampler():
    from torchao_fork_b200._models.llama.generate import Generator
    cfg = O.random_config(**CONFIGS["single"])
    m = _model(cfg, O.random_weights(cfg, seed=18), torch.bfloat16, slots=1, seq=32)
    gen = Generator(m, 1, 32, temperature=0.8, top_k=5)
    out = gen.generate(torch.tensor(_tokens(cfg, 5, 11)), 10)
    assert out.shape == (1, 15) and int(out.min()) >= 0 and int(out.max()) < cfg["vocab"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_on_a_checkpoint_folder(tmp_path, dtype):
    cfg = O.random_config(**CONFIGS["mixed"])
    w = O.random_weights(cfg, seed=19)
    O.write_checkpoint(str(tmp_path / "model"), cfg, w)
    a, b = _tokens(cfg, 26, 12), _tokens(cfg, 9, 13)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:22], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[22:], "want": [3]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "64", "--slots", "1"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    assert not (out / "1.f32").exists()
    ra, rb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    tol = F32_TOL if dtype == "float32" else max(_bf16_tol(cfg, w, a), _bf16_tol(cfg, w, b))
    V = cfg["vocab"]
    assert _err(np.fromfile(out / "0.f32", "<f4").reshape(-1, V), ra[[0, 19]]) < tol
    assert _err(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), ra[[25]]) < tol
    assert _err(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), rb[[8]]) < tol
