"""Tadolix, host side (no GPU): configuration reader and round trip, registry, checkpoint container, distance-bias table,
tile tables of the recurrences and of the chunked attention, state classes, and the oracle against an incremental
(token by token, with explicit state) restatement of itself."""
import math

import numpy as np
import pytest
import torch

import tadolix_oracle as O
from torchao_fork_b200._models import registry
from torchao_fork_b200._models.cache import ConvState, RecurrentState, RingKVCache, SequenceStates
from torchao_fork_b200._models.checkpoint import read_config, read_safetensors
from torchao_fork_b200._models.tadolix.model import TadolixArgs, distance_bias_table, tadolix_configs
from torchao_fork_b200._models.tadolix.step import chunk_tiles, scan_tiles, segments_of


def _cfg():
    return O.make_config([O.recurrent_layer(24, 3, 3, ff=40), O.attention_layer(), O.recurrent_layer(20, 1, 2),
                          O.attention_layer(heads=2, kv_heads=2, dim=16, vdim=8, chunk=5, rows=7, ff=0)],
                         width=32, streams=3, taps=3, loop=(1, 3, 2))


def test_config_reader_round_trip_and_layer_runs():
    cfg = O.clean_config(_cfg())
    a = TadolixArgs.from_dict(cfg)
    assert a.runs == O.layer_runs(cfg) == [0, 1, 2, 1, 2, 3]
    assert TadolixArgs.from_dict(a.to_dict()) == a
    assert a.layers[1].mixer.left.chunk == 8 and a.layers[3].mixer.left.kv_heads == 2 and a.layers[2].ff == 0
    assert a.streams == 3 and a.canon_taps == 3 and a.loop == (1, 3, 2)


def test_config_without_optional_parts():
    cfg = O.clean_config(O.make_config([O.attention_layer()], streams=0, taps=0))
    del cfg["layers"][0]["mixer"]["left"]["softcap"]
    a = TadolixArgs.from_dict(cfg)
    assert a.streams == 0 and a.canon_taps == 0 and a.loop is None and a.runs == [0]
    assert a.layers[0].mixer.left.softcap == 0.0


def test_unknown_mixer_is_refused():
    cfg = O.clean_config(_cfg())
    cfg["layers"][0]["type"] = "something"
    with pytest.raises(NotImplementedError):
        TadolixArgs.from_dict(cfg)


def test_registry_knows_the_family_and_its_names(tmp_path):
    fams = registry.families()
    assert "tadolix" in fams and set(tadolix_configs) <= set(fams["tadolix"].names())
    cfg = _cfg()
    O.write_checkpoint(str(tmp_path), cfg, O.random_weights(cfg))
    assert registry.architecture_of(str(tmp_path)) == "Tadolix"
    w = read_safetensors(str(tmp_path / "model.safetensors"))
    assert w["l1.mix.left.rel"].shape == (6, 4) and w["l0.mix.ra"].shape == (3, 8, 8) and w["l1.hc2.mix"].shape == (3, 3)
    assert "_rel_rows" not in read_config(str(tmp_path))["layers"][1]["mixer"]


@pytest.mark.parametrize("B,D", [(16, 100), (6, 20), (7, 33), (2, 9), (32, 128), (16, 128)])
def test_distance_bias_table_is_the_bucket_function(B, D):
    rel = torch.arange(B * 3, dtype=torch.float32).view(B, 3)
    n = 3 * D
    tab = distance_bias_table(rel, D, n)
    assert tab.shape == (3, n)
    for dist in range(n):
        assert torch.equal(tab[:, dist], rel[O.distance_bucket(dist, B, D)]), dist
    # one row per distance below B // 2, the last row from bias_max on, never decreasing in between
    rows = (tab[0] / 3).long().tolist()
    assert rows[: B // 2] == list(range(B // 2)) and rows[D] == B - 1 and rows == sorted(rows)


def test_segments_and_scan_tiles():
    slot = np.array([3, 3, 3, 3, 3, 1, 0, 0, 0], np.int32)
    pos = np.array([7, 8, 9, 10, 11, 40, 0, 1, 2], np.int32)
    starts, counts = segments_of(slot, pos)
    assert starts.tolist() == [0, 5, 6] and counts.tolist() == [5, 1, 3]
    first, count, seg0, segn = scan_tiles(starts, counts, 8)
    assert first.tolist() == [0, 5, 6] and count.tolist() == [5, 1, 3] and seg0 is None and segn is None
    first, count, seg0, segn = scan_tiles(starts, counts, 2)
    assert first.tolist() == [0, 2, 4, 5, 6, 8] and count.tolist() == [2, 2, 1, 1, 2, 1]
    assert seg0.tolist() == [0, 3, 4] and segn.tolist() == [3, 1, 2]
    # the same slot twice with a gap in positions is two segments
    s2, c2 = segments_of(np.array([1, 1, 1], np.int32), np.array([4, 5, 9], np.int32))
    assert s2.tolist() == [0, 2] and c2.tolist() == [2, 1]


@pytest.mark.parametrize("tile_rows,chunk", [(4, 8), (16, 5), (3, 3), (8, 1), (2, 64)])
def test_chunk_tiles_stay_inside_one_chunk_and_cover_every_row(tile_rows, chunk):
    slot = np.concatenate([np.full(23, 2), np.full(1, 0), np.full(9, 1)]).astype(np.int32)
    pos = np.concatenate([np.arange(6, 29), [17], np.arange(0, 9)]).astype(np.int32)
    starts, counts = segments_of(slot, pos)
    first, count = chunk_tiles(starts, counts, pos, tile_rows, chunk)
    covered = []
    for f, c in zip(first, count):
        assert 1 <= c <= tile_rows
        rows = list(range(f, f + c))
        assert len({int(slot[r]) for r in rows}) == 1 and len({int(pos[r]) // chunk for r in rows}) == 1
        covered += rows
    assert covered == list(range(len(slot)))


def test_state_classes_grow_and_keep_their_rows():
    ring, rec, conv = RingKVCache(2, 5, 3, 4, 6, torch.float32), RecurrentState(2, 7), ConvState(2, 4, 9)
    assert ring.k.shape == (2, 5, 3, 4) and ring.v.shape == (2, 5, 3, 6) and rec.s.shape == (2, 7) and conv.x.shape == (2, 3, 9)
    ring.k[1] = 1.0
    rec.s[0] = 2.0
    conv.x[1] = 3.0
    st = SequenceStates(2, 100)
    st.on_grow += [ring.grow, rec.grow, conv.grow]
    a, b = st.slot_of("a"), st.slot_of("b")
    c = st.slot_of("c")
    assert (a, b, c) == (0, 1, 2) and ring.k.shape[0] == 4 and rec.s.shape[0] == 4 and conv.x.shape[0] == 4
    assert float(ring.k[1].min()) == 1.0 and float(rec.s[0].min()) == 2.0 and float(conv.x[1].min()) == 3.0
    assert float(ring.k[2:].abs().max()) == 0.0
    st.release("a")
    assert st.slot_of("d") == 0 and st.length[0] == 0


# ------------------------------------------------------------------------------------------------ the oracle against itself
def _incremental(cfg, w, tokens):
    """The same model token by token with explicit state (last inputs of every convolution, recurrence states, the
    keys and values of the current chunk), written independently of the whole-sequence functions."""
    eps, S = cfg["norm"]["eps"], cfg.get("streams")
    W = cfg["width"]
    runs = O.layer_runs(cfg)
    F = O.F64
    g = lambda n: w[n].to(F)
    state = [dict(canon=[], conv=[], S=None, keys=[], vals=[]) for _ in runs]
    out = []
    for p, tok in enumerate(tokens):
        x0 = g("embed")[tok] * cfg["embedding"]["scale"]
        for i in range(W):
            f = 10000.0 ** (-2.0 * (i // 2) / W)
            x0[i] += math.sin(p * f) if i % 2 == 0 else math.cos(p * f)
        xs = [x0.clone() for _ in range(S or 1)]
        for r, li in enumerate(runs):
            lay, pre, s = cfg["layers"][li], f"l{li}.", state[r]
            for q in (1, 2):
                if q == 2 and not lay.get("mlp"):
                    continue
                u = sum(g(f"{pre}hc{q}.in")[k] * xs[k] for k in range(S)) if S else xs[0]
                h = u / torch.sqrt((u * u).mean() + eps) * (1 + g(f"{pre}norm{q}"))
                if q == 1:
                    if cfg.get("canon"):
                        taps, cw = cfg["canon"]["taps"], g(pre + "canon1")
                        hist = (s["canon"] + [h])[-taps:]
                        conv = sum(cw[:, taps - len(hist) + j] * hist[j] for j in range(len(hist)))
                        s["canon"] = hist
                        h = h + conv
                    m = lay["mixer"]
                    if lay["type"] == "parallel":
                        a, lp, rp = m["left"], pre + "mix.left.", pre + "mix.right."
                        H, G, d, dv, C = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
                        qv = (g(lp + "q") @ h).view(H, d)
                        kv = (g(lp + "k") @ h).view(G, d)
                        vv = (g(lp + "v") @ h).view(G, dv)
                        qv = qv / torch.sqrt((qv * qv).mean(-1, keepdim=True) + eps)
                        kv = kv / torch.sqrt((kv * kv).mean(-1, keepdim=True) + eps)
                        if p % C == 0:
                            s["keys"], s["vals"] = [], []
                        s["keys"].append(kv)
                        s["vals"].append(vv)
                        rel, res = g(lp + "rel"), []
                        for hd in range(H):
                            kh = hd // (H // G)
                            sc = torch.stack([(k_[kh] @ qv[hd]) * a["scale"] for k_ in s["keys"]])
                            if a["softcap"]:
                                sc = a["softcap"] * torch.tanh(sc / a["softcap"])
                            nk = len(s["keys"])
                            sc = sc + torch.stack([rel[O.distance_bucket(nk - 1 - j, rel.shape[0], a["bias_max"]), hd] for j in range(nk)])
                            pw = torch.softmax(sc, 0)
                            res.append(sum(pw[j] * s["vals"][j][kh] for j in range(nk)))
                        left = g(lp + "o") @ (torch.cat(res) * torch.sigmoid(g(lp + "g") @ h))
                        z = torch.sigmoid(g(rp + "z") @ h + g(rp + "z.b"))
                        uu = g(rp + "x") @ h + g(rp + "x.b")
                        cand = torch.where(uu >= 0, uu + 0.5, torch.sigmoid(uu))
                        s["S"] = z * cand if s["S"] is None else (1 - z) * s["S"] + z * cand
                        gg = g(rp + "g") @ h
                        right = g(rp + "o") @ (s["S"] * gg * torch.sigmoid(gg))
                        y = m["left_scale"] * left + m["right_scale"] * right
                    else:
                        mp, nb = pre + "mix.", m["blocks"]
                        yb = O.gelu_tanh(g(mp + "y") @ h + g(mp + "y.b"))
                        xb = g(mp + "x") @ h + g(mp + "x.b")
                        cw, taps = g(mp + "conv"), m["conv"]
                        hist = (s["conv"] + [xb])[-taps:]
                        s["conv"] = hist
                        uu = sum(cw[:, taps - len(hist) + j] * hist[j] for j in range(len(hist))) + g(mp + "conv.b")
                        bw = uu.shape[0] // nb
                        rr = torch.cat([g(mp + "ra")[b] @ uu[b * bw:(b + 1) * bw] for b in range(nb)]) + g(mp + "ra.b").reshape(-1)
                        ii = torch.cat([g(mp + "ri")[b] @ uu[b * bw:(b + 1) * bw] for b in range(nb)]) + g(mp + "ri.b").reshape(-1)
                        aa = torch.exp(-8.0 * torch.sigmoid(rr) * torch.log1p(torch.exp(g(mp + "lam"))))
                        bb = torch.sqrt(1 - aa * aa) * torch.sigmoid(ii) * uu
                        s["S"] = bb if s["S"] is None else aa * s["S"] + bb
                        y = g(mp + "o") @ (s["S"] * yb)
                else:
                    y = g(pre + "mlp.down") @ (O.gelu_tanh(g(pre + "mlp.gate") @ h) * (g(pre + "mlp.up") @ h))
                if S:
                    mix, co = g(f"{pre}hc{q}.mix"), g(f"{pre}hc{q}.out")
                    xs = [sum(mix[k, t] * xs[k] for k in range(S)) + co[t] * y for t in range(S)]
                else:
                    xs = [xs[0] + y]
        x = sum(xs)
        out.append(g("head") @ (x / torch.sqrt((x * x).mean() + eps) * (1 + g("final.norm"))))
    return torch.stack(out)


@pytest.mark.parametrize("plain", [False, True])
def test_oracle_whole_sequence_equals_token_by_token(plain):
    if plain:
        cfg = O.make_config([O.attention_layer(chunk=4, kv_heads=1, heads=3, softcap=0.0, ff=0), O.recurrent_layer(16, 2, 4, ff=24)],
                            width=20, streams=0, taps=0)
    else:
        cfg = _cfg()
    w = O.random_weights(cfg, seed=3)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = O.forward(cfg, w, toks), _incremental(cfg, w, toks)
    assert torch.allclose(a, b, rtol=1e-9, atol=1e-9)


def test_oracle_mechanisms_at_their_edges():
    # convolution: the last column meets the current row, zeros in front of the sequence
    x = torch.arange(1.0, 5.0, dtype=O.F64).view(4, 1)
    k = torch.tensor([[100.0, 10.0, 1.0]], dtype=O.F64)
    assert O.causal_conv(x, k).view(-1).tolist() == [1.0, 12.0, 123.0, 234.0]
    # buckets: exact below half, last bucket from bias_max on
    assert [O.distance_bucket(n, 8, 16) for n in (0, 3, 4, 15, 16, 1000)] == [0, 3, 4, 7, 7, 7]
    # a query in a new chunk does not see the chunk before: with chunk 1 the attention returns each row's own value
    a = O.attention_layer(heads=2, kv_heads=1, dim=4, vdim=4, chunk=1)["mixer"]["left"]
    cfg = O.make_config([O.attention_layer(heads=2, kv_heads=1, dim=4, vdim=4, chunk=1)], width=8)
    w = {k_: v.double() for k_, v in O.random_weights(cfg).items()}
    w["l0.mix.left.o"] = torch.eye(8, dtype=O.F64)
    h = torch.randn(5, 8, dtype=O.F64, generator=torch.Generator().manual_seed(0))
    got = O.chunk_attention(h, w, "l0.mix.left.", a, 1e-6)
    v = (h @ w["l0.mix.left.v"].T).repeat(1, 2) * torch.sigmoid(h @ w["l0.mix.left.g"].T)
    assert torch.allclose(got, v, atol=1e-12)
