"""Bitipel: a decoder-only language model built from
  * an fp32 residual stream, x <- x + m * norm(sublayer(x)) with the RMS norm (ONE learned number as weight) on the
    sublayer's OUTPUT,
  * a token shift in front of every mixer (the mixer's input is blended with the previous token's, per coordinate),
  * latent attention: queries per head with an unrotated and a rotated part, ONE compressed key/value row per token
    (a normed latent + a rotated key part shared by all heads) from which keys and values are up-projected per head,
    a softmax whose denominator also holds a learned per-head sink, a sigmoid output gate per head; a layer may reuse
    an earlier layer's cached rows instead of projecting its own,
  * a mixture of clipped-GLU experts (softmax router, top-k, scores not renormalised) plus a shared expert,
  * a learned weighted average over the embedding output and ALL layer results so far after every layer.

This module holds the configuration (read from a checkpoint's config.json: every size and constant comes from there),
the weights in the layout the kernels want, and the per-sequence state (cache.py).  The compute is step.py.
Checkpoint tensor names: embed, head, final.norm, l<i>.{norm1,norm2,shift,dwa}, l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,g,o},
l<i>.mlp.{router,e<k>.{gate,up,down},shared.{gate,up,down}}; linear weights are [out][in].
"""
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..cache import LatentKVCache, SequenceStates, TokenShiftState
from ..checkpoint import read_config, read_safetensors

GLU_ALPHA = 1.702   # slope inside the sigmoid of the experts' activation: fixed by the design


@dataclass
class LatentAttentionArgs:
    heads: int
    dim: int            # unrotated query / key size per head
    rot_dim: int        # rotated query / key size per head (the key part is shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int       # how many of the rot_dim coordinates rotate (pairs 2i, 2i+1)
    kv_from: Optional[int] = None   # layer whose cached rows this layer attends over (None: its own)


@dataclass
class MoEArgs:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int = 0          # 0: no shared expert
    shared_limit: float = 0.0


@dataclass
class LayerArgs:
    mixer: LatentAttentionArgs
    mlp: Optional[MoEArgs]


@dataclass
class BitipelArgs:
    vocab_size: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: List[LayerArgs] = field(default_factory=list)
    block_size: int = 1 << 30   # the design has no built-in context limit; the caches set it

    @property
    def n_layer(self):
        return len(self.layers)

    @classmethod
    def from_dict(cls, cfg: dict) -> "BitipelArgs":
        layers = []
        for i, lay in enumerate(cfg["layers"]):
            if lay.get("type", "latent_attention") != "latent_attention":
                raise NotImplementedError(f"layer {i}: mixer type {lay.get('type')!r}")
            m = lay["mixer"]
            rot = m.get("rot") or {}
            mixer = LatentAttentionArgs(
                heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot_base=float(rot.get("base", 10000.0)),
                rot_dims=int(rot.get("dims", m["rot_dim"])), kv_from=(int(m["kv_from"]) if m.get("kv_from") is not None else None))
            mlp = None
            if lay.get("mlp"):
                f = lay["mlp"]
                if f.get("kind", "moe") != "moe":
                    raise NotImplementedError(f"layer {i}: feed-forward kind {f.get('kind')!r}")
                sh = f.get("shared") or {}
                mlp = MoEArgs(experts=int(f["router"]["experts"]), top=int(f["router"]["top"]), ff=int(f["expert"]["ff"]),
                              limit=float(f["expert"]["limit"]), shared_ff=int(sh.get("ff", 0)),
                              shared_limit=float(sh.get("limit", 0.0)))
            layers.append(LayerArgs(mixer, mlp))
        for i, lay in enumerate(layers):
            j = lay.mixer.kv_from
            if j is not None:
                src = layers[j].mixer
                assert 0 <= j < i and src.kv_from is None, f"layer {i}: kv_from {j} must name an earlier layer with its own latents"
                assert (src.kv_rank, src.rot_dim) == (lay.mixer.kv_rank, lay.mixer.rot_dim)
        return cls(vocab_size=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]),
                   residual_mult=float(cfg["residual_mult"]), layers=layers)

    def to_dict(self) -> dict:
        out = []
        for lay in self.layers:
            m = lay.mixer
            mx = {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "rot": {"base": m.rot_base, "dims": m.rot_dims},
                  "rot_dim": m.rot_dim, "scale": m.scale, "vdim": m.vdim}
            if m.kv_from is not None:
                mx["kv_from"] = m.kv_from
            f = lay.mlp
            mlp = None if f is None else {
                "expert": {"ff": f.ff, "limit": f.limit}, "kind": "moe", "router": {"experts": f.experts, "top": f.top},
                **({"shared": {"ff": f.shared_ff, "limit": f.shared_limit}} if f.shared_ff else {})}
            out.append({"mixer": mx, "mlp": mlp, "type": "latent_attention"})
        return {"architecture": "Bitipel", "layers": out, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "vocab": self.vocab_size, "width": self.width}


def _stack(n_layer, width, heads, dim, rot_dim, vdim, kv_rank, experts, top, ff, shared_ff, vocab, share_every=2):
    """n_layer equal layers; every `share_every`-th layer projects its own latents, the ones between reuse them."""
    layers = []
    for i in range(n_layer):
        own = i % share_every == 0
        layers.append(LayerArgs(
            LatentAttentionArgs(heads, dim, rot_dim, vdim, kv_rank, 1.0 / math.sqrt(dim + rot_dim), 500000.0, rot_dim,
                                None if own else i - i % share_every),
            MoEArgs(experts, top, ff, 7.0, shared_ff, 7.0)))
    return BitipelArgs(vocab, width, 1e-5, 0.7, layers)


# named random-init configurations (benchmarks and examples; checkpoints carry their own config.json)
bitipel_configs = {
    "Bitipel-test": lambda: _stack(4, 128, 4, 16, 8, 24, 64, 6, 2, 48, 64, 512),
    # layers of the size of a 1-2 B parameter model / of a 7-8 B parameter model (4 layers each: a layer benchmark)
    "Bitipel-2k": lambda: _stack(4, 2048, 16, 128, 64, 128, 512, 32, 4, 1024, 2048, 32000),
    "Bitipel-4k": lambda: _stack(4, 4096, 32, 128, 64, 128, 512, 64, 6, 1408, 2816, 128256),
}


class _Layer:
    """One layer's tensors as the kernels read them (plain attributes; the module registers them as buffers)."""


class Bitipel(nn.Module):
    def __init__(self, config: BitipelArgs, weights: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32), "Bitipel runs in bfloat16 or float32"
        self.config, self.dtype = config, dtype
        self.device = torch.device(device)
        self.max_batch_size = -1
        self.max_seq_length = -1
        self.states: Optional[SequenceStates] = None
        self._step = None
        self._take(weights)

    # ------------------------------------------------------------------------------------------------ weights
    def _take(self, w: Dict[str, torch.Tensor]):
        cfg, dev, dt = self.config, self.device, self.dtype
        used = set()

        def get(name, shape=None):
            if name not in w:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = w[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, the configuration asks for {tuple(shape)}")
            return t.to(device=dev, dtype=dt)

        def buf(name, t):
            self.register_buffer(name.replace(".", "__"), t.contiguous(), persistent=False)
            return getattr(self, name.replace(".", "__"))

        W, V = cfg.width, cfg.vocab_size
        self.embed = buf("embed", get("embed", (V, W)))
        self.head = buf("head", get("head", (V, W)))
        self.final_norm = buf("final.norm", get("final.norm").reshape(1))
        self.layers: List[_Layer] = []
        for i, la in enumerate(cfg.layers):
            m, p, L = la.mixer, f"l{i}.", _Layer()
            H, dn, dr, dv, R = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
            L.args = la
            L.norm1 = buf(p + "norm1", get(p + "norm1").reshape(1))
            L.shift = buf(p + "shift", get(p + "shift", (W,)))
            L.dwa = buf(p + "dwa", get(p + "dwa", (i + 2,)))
            parts = [get(p + "mix.q", (H * (dn + dr), W))]
            L.q_off, L.kv_off = 0, -1
            if m.kv_from is None:
                L.kv_off = parts[0].shape[0]
                parts.append(get(p + "mix.dkv", (R + dr, W)))
                L.c_norm = buf(p + "mix.dkv.norm", get(p + "mix.dkv.norm", (R,)))
            else:
                L.c_norm = None
            L.g_off = sum(t.shape[0] for t in parts)
            parts.append(get(p + "mix.g", (H, W)))
            L.w_in = buf(p + "mix.in", torch.cat(parts, 0))                      # [q | dkv | gate][W]: one GEMM
            L.uk = buf(p + "mix.uk", get(p + "mix.uk", (H * dn, R)).view(H, dn, R))   # q_abs[h] = q_n[h] @ uk[h]
            L.uvT = buf(p + "mix.uvT", get(p + "mix.uv", (H * dv, R)).view(H, dv, R).transpose(1, 2))   # [H][R][dv]
            # the same two matrices as [R][H dn] / [R][H dv] operands: keys and values of a whole prompt in one GEMM each
            L.ukx = L.uk.view(H * dn, R)
            L.uvx = buf(p + "mix.uvx", get(p + "mix.uv", (H * dv, R)).t())
            L.sink = buf(p + "mix.sink", get(p + "mix.sink", (H,)))
            L.o = buf(p + "mix.o", get(p + "mix.o", (W, H * dv)))
            half = m.rot_dims // 2
            freq = torch.tensor([m.rot_base ** (-2.0 * j / m.rot_dims) for j in range(half)], dtype=torch.float64)
            L.inv_freq = buf(p + "mix.inv_freq", freq.to(torch.float32).to(dev))
            f = la.mlp
            if f is not None:
                L.norm2 = buf(p + "norm2", get(p + "norm2").reshape(1))
                L.router = buf(p + "mlp.router", get(p + "mlp.router", (f.experts, W)))
                L.wgu = buf(p + "mlp.wgu", torch.stack([torch.cat([get(f"{p}mlp.e{e}.gate", (f.ff, W)), get(f"{p}mlp.e{e}.up", (f.ff, W))], 0)
                                                        for e in range(f.experts)]))            # [E][2 ff][W]
                L.wd = buf(p + "mlp.wd", torch.stack([get(f"{p}mlp.e{e}.down", (W, f.ff)) for e in range(f.experts)]))
                if f.shared_ff:
                    L.sgu = buf(p + "mlp.sgu", torch.cat([get(p + "mlp.shared.gate", (f.shared_ff, W)),
                                                          get(p + "mlp.shared.up", (f.shared_ff, W))], 0))
                    L.sd = buf(p + "mlp.sd", get(p + "mlp.shared.down", (W, f.shared_ff)))
            self.layers.append(L)
        extra = sorted(set(w) - used)
        if extra:
            raise ValueError(f"checkpoint tensors the configuration does not use: {extra[:8]}{' ...' if len(extra) > 8 else ''}")

    @classmethod
    def from_checkpoint(cls, folder, device="cuda", dtype=torch.bfloat16):
        import os
        cfg = BitipelArgs.from_dict(read_config(folder))
        return cls(cfg, read_safetensors(os.path.join(str(folder), "model.safetensors")), device, dtype).eval()

    @classmethod
    def from_name(cls, name, device="cuda", dtype=torch.bfloat16):
        return cls.random_init(bitipel_configs[name](), device, dtype)

    @classmethod
    def random_init(cls, cfg: BitipelArgs, device="cuda", dtype=torch.bfloat16, seed=1234):
        """Seeded random weights of every tensor the configuration names (no checkpoints exist offline), drawn on `device`."""
        g = torch.Generator(device=device).manual_seed(seed)
        W = cfg.width

        def mat(o, i, s=1.0):
            return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * (s / math.sqrt(i))).to(dtype)

        def vec(n, mean=0.0, s=1.0):
            return (mean + s * torch.randn(n, generator=g, device=device, dtype=torch.float32)).to(dtype)

        w = {"embed": vec((cfg.vocab_size, W)), "head": mat(cfg.vocab_size, W), "final.norm": vec((), 1.0, 0.05)}
        for i, la in enumerate(cfg.layers):
            m, p = la.mixer, f"l{i}."
            w[p + "norm1"], w[p + "shift"] = vec((), 1.0, 0.1), torch.rand(W, generator=g, device=device).to(dtype)
            w[p + "dwa"] = (vec(i + 2, 0.0, 0.2).float() + 0.8 * (torch.arange(i + 2, device=device) == i + 1)).to(dtype)
            w[p + "mix.q"] = mat(m.heads * (m.dim + m.rot_dim), W, 2.0)
            if m.kv_from is None:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(m.kv_rank + m.rot_dim, W), vec(m.kv_rank, 1.0, 0.1)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(m.heads * m.dim, m.kv_rank, 2.0), mat(m.heads * m.vdim, m.kv_rank)
            w[p + "mix.sink"], w[p + "mix.g"], w[p + "mix.o"] = vec(m.heads), mat(m.heads, W, 2.0), mat(W, m.heads * m.vdim)
            f = la.mlp
            if f is not None:
                w[p + "norm2"], w[p + "mlp.router"] = vec((), 1.0, 0.1), mat(f.experts, W, 3.0)
                for e in range(f.experts):
                    w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(f.ff, W, 2.0), mat(f.ff, W, 2.0), mat(W, f.ff)
                if f.shared_ff:
                    w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"] = mat(f.shared_ff, W, 2.0), mat(f.shared_ff, W, 2.0)
                    w[p + "mlp.shared.down"] = mat(W, f.shared_ff)
        return cls(cfg, w, device, dtype).eval()

    def weight_bytes(self, ignore_embeddings=False) -> int:
        skip = {"embed"} if ignore_embeddings else set()
        return sum(b.numel() * b.element_size() for n, b in self.named_buffers() if n not in skip)

    # ------------------------------------------------------------------------------------------------ state
    def setup_caches(self, max_batch_size, max_seq_length, dtype=None, device=None, kv_cache_quantization=False):
        """Per-sequence state for `max_batch_size` slots of `max_seq_length` positions: a LatentKVCache in every layer
        that projects its own latents, a TokenShiftState in every layer.  Same call as the Llama's setup_caches."""
        if kv_cache_quantization:
            raise NotImplementedError("Bitipel keeps its latent rows in the model's dtype")
        if self.states is not None and self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        self.max_batch_size, self.max_seq_length = max_batch_size, max_seq_length
        self.states = SequenceStates(max_batch_size, max_seq_length)
        for L in self.layers:
            m = L.args.mixer
            L.kv_cache = LatentKVCache(max_batch_size, max_seq_length, m.kv_rank, m.rot_dim, self.dtype, self.device) \
                if m.kv_from is None else None
            L.shift_state = TokenShiftState(max_batch_size, self.config.width, self.device)
            self.states.on_grow.append(L.shift_state.grow)
            if L.kv_cache is not None:
                self.states.on_grow.append(L.kv_cache.grow)
        self.states.on_grow.append(lambda n: setattr(self, "max_batch_size", n))
        self._step = None

    @property
    def step_engine(self):
        """The step function over this model's weights and state (step.py), made on first use."""
        if self._step is None:
            from .step import StepEngine
            assert self.states is not None, "call setup_caches first"
            self._step = StepEngine(self)
        return self._step

    def make_decode_engine(self, batch_size, temperature=0.8, top_k=200, **unused):
        from .step import GraphDecodeEngine
        return GraphDecodeEngine(self, batch_size, temperature, top_k)

    @torch.no_grad()
    def forward(self, idx: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """idx [B][T] at positions input_pos [T] (default 0 .. T-1) of the sequences in slots 0 .. B-1 -> logits of the
        LAST position [B][1][vocab] in fp32 (what generation samples from).  The Llama's forward call shape."""
        assert self.states is not None, "Caches must be initialized first"
        B, T = idx.shape
        start = 0 if input_pos is None else int(input_pos[0])
        st = self.states
        segs = []
        for b in range(B):
            slot = st.slot_of(("batch", b))
            assert slot == b, "generation batches own slots 0 .. B-1: release other requests first"
            st.length[slot] = start          # generation writes where it is told to
            segs.append((slot, idx[b]))
        logits = self.step_engine.step(segs, want="last")
        return logits.view(B, 1, -1)
