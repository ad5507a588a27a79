"""Host-side parts of the Bitipel family that need no GPU: configuration reader, checkpoint container, registry, slot
allocator / state manager, attention tile tables, and the oracle's own consistency (whole sequence == incremental)."""
import json
import os

import numpy as np
import pytest
import torch

import bitipel_oracle as O
from torchao_fork_b200._models import registry
from torchao_fork_b200._models.bitipel import Bitipel, BitipelArgs, bitipel_configs
from torchao_fork_b200._models.cache import SequenceStates, SlotAllocator
from torchao_fork_b200._models.checkpoint import is_checkpoint_folder, read_safetensors


def test_config_round_trip_and_validation():
    cfg = O.random_config(n_layers=4, share=(None, 0, None, 2), no_mlp=(1,))
    args = BitipelArgs.from_dict(cfg)
    assert args.n_layer == 4 and args.layers[1].mlp is None and args.layers[3].mixer.kv_from == 2
    assert args.layers[0].mixer.rot_base == cfg["layers"][0]["mixer"]["rot"]["base"]
    assert BitipelArgs.from_dict(args.to_dict()) == args
    bad = O.random_config(n_layers=2, share=(None, 1))
    with pytest.raises(AssertionError):
        BitipelArgs.from_dict(bad)          # a layer cannot borrow from itself or a later layer
    for name, make in bitipel_configs.items():
        assert BitipelArgs.from_dict(make().to_dict()) == make(), name


def test_checkpoint_folder_reader_and_registry(tmp_path):
    cfg = O.random_config()
    w = O.random_weights(cfg, seed=3)
    O.write_checkpoint(str(tmp_path), cfg, w)
    assert is_checkpoint_folder(tmp_path) and registry.architecture_of(tmp_path) == "Bitipel"
    got = read_safetensors(tmp_path / "model.safetensors")
    assert set(got) == set(w)
    for k in w:
        assert got[k].dtype == w[k].dtype and got[k].shape == w[k].shape and torch.equal(got[k], w[k]), k
    model = registry.load_checkpoint_folder(tmp_path, device="cpu", dtype=torch.bfloat16)
    assert isinstance(model, Bitipel) and model.config == BitipelArgs.from_dict(cfg)
    lay = model.layers[1]                     # borrows layer 0's latents: no down projection of its own
    m = cfg["layers"][1]["mixer"]
    assert lay.kv_off == -1 and lay.w_in.shape[0] == m["heads"] * (m["dim"] + m["rot_dim"]) + m["heads"]
    assert torch.equal(model.layers[0].w_in[: lay.g_off - 0][: m["heads"] * (m["dim"] + m["rot_dim"])], w["l0.mix.q"])
    # a tensor that the configuration does not name is an error, and so is a missing one
    w2 = dict(w)
    w2["l0.mix.extra"] = torch.zeros(1, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        Bitipel(BitipelArgs.from_dict(cfg), w2, "cpu")
    w3 = {k: v for k, v in w.items() if k != "l2.mix.dkv"}
    with pytest.raises(KeyError):
        Bitipel(BitipelArgs.from_dict(cfg), w3, "cpu")
    assert "Bitipel-test" in registry.families()["bitipel"].names() and "Llama-3-8B" in registry.families()["llama"].names()


def test_slots_are_reused_lowest_first_and_grow():
    a = SlotAllocator(3)
    assert [a.alloc(), a.alloc(), a.alloc()] == [0, 1, 2]
    with pytest.raises(RuntimeError):
        a.alloc()
    a.free(1)
    a.free(0)
    assert a.alloc() == 0 and a.in_use == 2
    st = SequenceStates(2, 10)
    grown = []
    st.on_grow.append(grown.append)
    assert st.slot_of("a") == 0 and st.slot_of("b") == 1 and st.slot_of("a") == 0
    assert st.extend(0, 4) == 0 and st.extend(0, 3) == 4 and st.length[0] == 7
    with pytest.raises(RuntimeError):
        st.extend(0, 4)                        # 11 positions do not fit 10
    assert st.slot_of("c") == 2 and grown == [4]
    st.release("a")
    assert st.slot_of("d") == 0 and st.length[0] == 0     # a freed slot starts over


def test_attention_tiles_follow_sequences():
    from torchao_fork_b200._models.bitipel.step import StepEngine
    slot = np.array([0, 0, 0, 0, 0, 1, 2, 2, 2], np.int32)
    pos = np.array([7, 8, 9, 10, 11, 0, 3, 4, 5], np.int32)
    first, count = StepEngine._tiles(None, slot, pos, 2)
    assert first.tolist() == [0, 2, 4, 5, 6, 8] and count.tolist() == [2, 2, 1, 1, 2, 1]
    first, count = StepEngine._tiles(None, slot, pos, 8)
    assert first.tolist() == [0, 5, 6] and count.tolist() == [5, 1, 3]
    first, count = StepEngine._tiles(None, slot[:1], pos[:1], 4)
    assert first.tolist() == [0] and count.tolist() == [1]


def test_expanded_attention_plan_tiles_key_rows_and_threshold():
    """Which steps attend in the expanded form, and where each sequence's keys go in the step's key / value buffers."""
    from types import SimpleNamespace
    from torchao_fork_b200._models.bitipel import step as S
    from torchao_fork_b200._models.bitipel.step import StepEngine
    cfg = bitipel_configs["Bitipel-test"]()
    eng = SimpleNamespace(expand_tile=4, cfg=cfg)
    # two sequences: 40 tokens from position 10, 35 tokens from position 0
    slot = np.concatenate([np.full(40, 3), np.full(35, 1)]).astype(np.int32)
    pos = np.concatenate([np.arange(10, 50), np.arange(35)]).astype(np.int32)
    (first, count, row), hist, rows = StepEngine._expand_plan(eng, slot, pos)
    assert hist == [(3, 50, 0), (1, 35, 50)] and rows == 85          # keys 0 .. last position of each, one after the other
    assert first.tolist() == list(range(0, 40, 4)) + list(range(40, 75, 4))
    assert count.tolist() == [4] * 10 + [4] * 8 + [3]
    assert row.tolist() == [0] * 10 + [50] * 9
    # fewer tokens per sequence than the threshold: the folded form serves the step
    assert StepEngine._expand_plan(eng, slot[:S.EXPAND_MIN_TOKENS - 1], pos[:S.EXPAND_MIN_TOKENS - 1]) is None
    one_each = np.arange(40, dtype=np.int32)
    assert StepEngine._expand_plan(eng, one_each, np.zeros(40, np.int32)) is None
    # no shape of the model is covered by the kernel
    assert StepEngine._expand_plan(SimpleNamespace(expand_tile=0, cfg=cfg), slot, pos) is None


def test_oracle_whole_sequence_equals_incremental_restatement():
    """The oracle's forward sees the whole sequence; restating one layer position by position with explicit carried
    state (previous input row, cached latents) must give the same numbers — the two readings of the equations agree."""
    cfg = O.random_config(n_layers=2, share=(None, 0))
    w = O.random_weights(cfg, seed=5)
    toks = [3, 17, 9, 44, 2, 60]
    _, layers = O.forward(cfg, w, toks, return_layers=True)
    x = w["embed"].to(O.F64)[torch.tensor(toks)]
    mx, eps, m = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], cfg["residual_mult"]
    prev = torch.zeros(cfg["width"], dtype=O.F64)
    cs, krs, outs = [], [], []
    for t in range(len(toks)):
        h = O.token_shift(x[t:t + 1], w["l0.shift"].to(O.F64), prev)
        prev = x[t]
        c, kr = O.latent_kv(h, torch.tensor([t]), w, "l0.mix.", mx, eps)
        cs.append(c)
        krs.append(kr)
        a = O.latent_attention(h, torch.tensor([t]), torch.cat(cs), torch.cat(krs), w, "l0.mix.", mx)
        y = x[t:t + 1] + m * O.scalar_norm(a, w["l0.norm1"].to(O.F64), eps)
        y = y + m * O.scalar_norm(O.mixture(y, w, "l0.mlp.", cfg["layers"][0]["mlp"]), w["l0.norm2"].to(O.F64), eps)
        outs.append(O.depth_average([x[t:t + 1], y], w["l0.dwa"].to(O.F64)))
    assert torch.allclose(torch.cat(outs), layers[0], rtol=1e-10, atol=1e-10)
