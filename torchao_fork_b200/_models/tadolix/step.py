"""The step function of Tadolix: runs the tokens a step brings — any mix of prompt portions and single decoded tokens of
several sequences — through the model's layer runs on the state that earlier steps left, as launches of libao_b200_lm
kernels (include/ao_b200_lm.h) and library GEMMs for the dense projections.

Per sublayer: read-out of the streams + norm (`streams_norm`) -> [mixer only: causal convolution added to the input] ->
the sublayer -> write-back into the streams (`streams_update`, which also saves the convolution's memory).
  parallel mixer: ONE GEMM for [q | k | v | gate | z | x | gate of the recurrence] with an fp32 result -> `qk_prep` (unit-RMS
      queries and keys) -> `chunk_attention` over the ring cache and the step's own rows -> `ring_append` -> `mingru_scan`
      -> ONE GEMM over [attention result | recurrence result] with [W_o left | W_o right]: the two branch scales are
      applied by the kernels that write the operands, so the sum of the branches is the GEMM's own accumulation.
  rglru mixer: GEMM [y | x] (fp32) -> `causal_conv` -> batched GEMM of the block-diagonal gates -> `rglru_scan` (saves the
      convolution's memory too) -> GEMM W_o.
  feed-forward: GEMM [gate | up] -> `gelu_glu` -> GEMM down.
The streams, norms, gates, recurrences, attention scores and weights are fp32 in both storage types.

`StepEngine.step` is what prefill, the trace runner and tests call; `GraphDecodeEngine` wraps the same layer loop for
one token per sequence with all metadata in device memory, captured into a CUDA graph (the Llama DecodeEngine's role).
"""
import ctypes
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ... import _lib
from .model import RGLRU_DECAY, Tadolix

# a portion longer than this is cut into pieces (bounds the workspace)
MAX_STEP_TOKENS = 4096
# rows of a recurrence tile; a step whose segments all fit one tile scans in one launch
SCAN_TILE = 32
# steps that bring at least this many rows per sequence (on average) attend with the tensor-core kernel (bf16 models,
# head sizes it covers); decoded tokens and short portions use the fp32 kernel, which shares a key block between the
# few rows of a tile and all query heads of a key/value head
PROMPT_MIN_ROWS = 16


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class StepMeta:
    """Device-side description of a step's rows: per row slot / position / rows of its segment in front (back) and
    behind (ahead); tiles of the recurrences; tiles of every attention shape."""
    n: int
    slot: torch.Tensor
    pos: torch.Tensor
    back: torch.Tensor
    ahead: torch.Tensor
    scan: tuple          # (tile_first, tile_count, n_tiles, seg_tile0 | None, seg_tiles | None, n_segments)
    attn: Dict[tuple, tuple]   # attention shape -> (tile_first, tile_count, n_tiles, tensor-core form?)


def segments_of(slot: np.ndarray, pos: np.ndarray):
    """(first row, rows) of every run of consecutive positions of one sequence."""
    n = len(slot)
    brk = np.flatnonzero((slot[1:] != slot[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
    starts = np.concatenate([[0], brk]).astype(np.int64)
    ends = np.concatenate([brk, [n]]).astype(np.int64)
    return starts, ends - starts


def scan_tiles(starts: np.ndarray, counts: np.ndarray, tile: int):
    """Tiles of <= `tile` rows inside the segments, and per segment its first tile and tile count (None, None when
    every segment is one tile)."""
    first, count, seg0, segn = [], [], [], []
    for s, c in zip(starts, counts):
        f = np.arange(s, s + c, tile)
        seg0.append(len(first))
        segn.append(len(f))
        first += f.tolist()
        count += np.minimum(tile, s + c - f).tolist()
    first, count = np.asarray(first, np.int32), np.asarray(count, np.int32)
    if max(segn) == 1:
        return first, count, None, None
    return first, count, np.asarray(seg0, np.int32), np.asarray(segn, np.int32)


def chunk_tiles(starts: np.ndarray, counts: np.ndarray, pos: np.ndarray, tile_rows: int, chunk: int):
    """Runs of <= tile_rows rows of one segment that lie inside ONE chunk of the sequence's positions."""
    first, count = [], []
    for s, c in zip(starts, counts):
        r, end = int(s), int(s + c)
        while r < end:
            room = chunk - int(pos[r]) % chunk          # rows up to the chunk's end
            k = min(tile_rows, room, end - r)
            first.append(r)
            count.append(k)
            r += k
    return np.asarray(first, np.int32), np.asarray(count, np.int32)


class StepEngine:
    def __init__(self, model: Tadolix):
        assert model.device.type == "cuda", "Tadolix runs on CUDA only: there is no CPU path"
        self.m, self.cfg = model, model.config
        self.dev = model.device
        self.dt = _lib.DT_BF16 if model.dtype == torch.bfloat16 else _lib.DT_F32
        self.L = _lib.lm()
        if model.dtype == torch.float32:
            # true fp32 products: no TF32 / reduced-precision accumulation in the library GEMMs
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        self.launches = 0
        self.sm_count = torch.cuda.get_device_properties(self.dev).multi_processor_count
        # rows of one sequence that an attention CTA takes, per attention shape of the model
        self.attn_keys, self.prompt_keys = {}, {}
        for la in self.cfg.layers:
            if la.type != "parallel":
                continue
            a = la.mixer.left
            tr = ctypes.c_int()
            _lib.lm_check(self.L.ao_lm_chunk_attention_plan(self.dt, a.heads, a.kv_heads, a.dim, a.vdim, ctypes.byref(tr)),
                          "chunk_attention_plan")
            if tr.value <= 0:
                raise NotImplementedError(f"attention shape not covered by the kernels: {a}")
            self.attn_keys[(a.heads, a.kv_heads, a.dim, a.vdim, a.chunk)] = (tr.value, a.chunk, False)
            _lib.lm_check(self.L.ao_lm_chunk_attention_prompt_plan(self.dt, a.heads, a.kv_heads, a.dim, a.vdim, ctypes.byref(tr)),
                          "chunk_attention_prompt_plan")
            if tr.value > 0:
                self.prompt_keys[(a.heads, a.kv_heads, a.dim, a.vdim, a.chunk)] = (tr.value, a.chunk, True)

    # ------------------------------------------------------------------------------------------------ public
    @torch.no_grad()
    def step(self, segments: Sequence[Tuple[int, Union[torch.Tensor, Sequence[int]]]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """segments: [(slot, tokens)] — the next tokens of the sequences in those slots (each slot at most once).
        want: "last" (the last token of every segment), "all", or per segment the indices among ITS tokens.
        Returns fp32 logits [wanted][vocab] in segment order.  Positions continue from the state manager's lengths."""
        st = self.m.states
        toks, slots, poss, rows = [], [], [], []
        at = 0
        seen = set()
        for k, (slot, t) in enumerate(segments):
            t = torch.as_tensor(t).reshape(-1).to(torch.int64).cpu().numpy() if not isinstance(t, np.ndarray) else t.astype(np.int64)
            n = len(t)
            assert n > 0 and slot not in seen, "every slot at most once per step, with at least one token"
            seen.add(slot)
            p0 = st.extend(slot, n)
            toks.append(t)
            slots.append(np.full(n, slot, np.int32))
            poss.append(np.arange(p0, p0 + n, dtype=np.int32))
            sel = [n - 1] if want == "last" else list(range(n)) if want == "all" else list(want[k])
            rows += [at + int(i) for i in sel]
            at += n
        tok, slot, pos = np.concatenate(toks), np.concatenate(slots), np.concatenate(poss)
        if (tok < 0).any() or (tok >= self.cfg.vocab_size).any():
            raise ValueError("token id outside the vocabulary")
        total = at
        if total <= MAX_STEP_TOKENS:
            x = self._run(tok, slot, pos)
            return self._logits(x, rows)
        # long portions: pieces of at most MAX_STEP_TOKENS tokens, in order (a piece may end inside a segment; the state
        # that a piece leaves is what the next one starts from, exactly as between steps)
        rows_np = np.asarray(rows, np.int64)
        result = torch.empty(len(rows), self.cfg.vocab_size, dtype=torch.float32, device=self.dev)
        for lo in range(0, total, MAX_STEP_TOKENS):
            hi = min(total, lo + MAX_STEP_TOKENS)
            x = self._run(tok[lo:hi], slot[lo:hi], pos[lo:hi])
            where = np.flatnonzero((rows_np >= lo) & (rows_np < hi))     # wanted rows keep the order they were asked in
            if len(where):
                result[torch.from_numpy(where).to(self.dev)] = self._logits(x, (rows_np[where] - lo).tolist())
        return result

    # ------------------------------------------------------------------------------------------------ pieces
    def _meta(self, slot: np.ndarray, pos: np.ndarray, tok: np.ndarray):
        """All of a piece's metadata in ONE host-to-device copy -> (device tokens, StepMeta)."""
        n = len(slot)
        starts, counts = segments_of(slot, pos)
        back, ahead = np.empty(n, np.int32), np.empty(n, np.int32)
        for s, c in zip(starts, counts):
            back[s:s + c] = np.arange(c)
            ahead[s:s + c] = np.arange(c - 1, -1, -1)
        sf, sc, seg0, segn = scan_tiles(starts, counts, SCAN_TILE)
        parts = [tok.view(np.int32), slot, pos, back, ahead, sf, sc]
        if seg0 is not None:
            parts += [seg0, segn]
        attn_np = {}
        prompt = n >= PROMPT_MIN_ROWS * len(starts)
        meta_shapes = {shape: (self.prompt_keys[shape] if prompt and shape in self.prompt_keys else key)
                       for shape, key in self.attn_keys.items()}
        for key in sorted(set(meta_shapes.values())):
            attn_np[key] = chunk_tiles(starts, counts, pos, key[0], key[1])
            parts += list(attn_np[key])
        packed = torch.from_numpy(np.concatenate(parts)).to(self.dev, non_blocking=True)
        o = [0]

        def take(k):
            v = packed[o[0]:o[0] + k]
            o[0] += k
            return v

        d_tok = take(2 * n).view(torch.int64)
        meta = StepMeta()
        meta.n = n
        meta.slot, meta.pos, meta.back, meta.ahead = take(n), take(n), take(n), take(n)
        nt = len(sf)
        tf, tc = take(nt), take(nt)
        if seg0 is not None:
            meta.scan = (tf, tc, nt, take(len(seg0)), take(len(seg0)), len(seg0))
        else:
            meta.scan = (tf, tc, nt, None, None, 0)
        tables = {}
        for key in sorted(attn_np):
            k = len(attn_np[key][0])
            tables[key] = (take(k), take(k), k, key[2])
        meta.attn = {shape: tables[key] for shape, key in meta_shapes.items()}
        return d_tok, meta

    def _run(self, tok: np.ndarray, slot: np.ndarray, pos: np.ndarray) -> torch.Tensor:
        """One piece through all layer runs -> the streams [n][S][W], fp32."""
        d_tok, meta = self._meta(slot, pos, tok)
        return self._layers(d_tok, meta)

    def _layers(self, d_tok: torch.Tensor, meta: StepMeta, after_run=None) -> torch.Tensor:
        m, cfg, L, dt, dev = self.m, self.cfg, self.L, self.dt, self.dev
        n, W, S = meta.n, cfg.width, max(1, cfg.streams)
        st = torch.cuda.current_stream(dev).cuda_stream
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=m.dtype, device=dev)
        x = torch.empty(n, S, W, **f32)
        hn = torch.empty(n, W, **f32)
        h = torch.empty(n, W, **act)
        _lib.lm_check(L.ao_lm_embed_sinusoid(_p(m.embed), dt, _p(d_tok), _p(meta.pos), n, W, cfg.embedding_scale, _p(m.pos_freq),
                                             S, _p(x), st), "embed_sinusoid")
        launches = 1
        taps = cfg.canon_taps
        for r, li in enumerate(cfg.runs):
            lay, rs = m.layers[li], m.run_state[r]
            la = lay.args
            hc = lay.hc[0]
            # ---- mixer sublayer
            if taps:
                _lib.lm_check(L.ao_lm_streams_norm(_p(x), None, n, S, W, _p(hc[0]) if hc else None, _p(lay.norm[0]), dt, 1.0,
                                                   cfg.norm_eps, _p(hn), None, st), "streams_norm")
                _lib.lm_check(L.ao_lm_causal_conv(_p(hn), W, None, n, W, taps, _p(lay.canon), None, dt, 1, _p(rs.canon.x),
                                                  _p(meta.slot), _p(meta.pos), _p(meta.back), None, _p(h), st), "causal_conv")
                launches += 2
            else:
                _lib.lm_check(L.ao_lm_streams_norm(_p(x), None, n, S, W, _p(hc[0]) if hc else None, _p(lay.norm[0]), dt, 1.0,
                                                   cfg.norm_eps, None, _p(h), st), "streams_norm")
                launches += 1
            if la.type == "parallel":
                y, k = self._parallel(lay, la.mixer, rs, h, meta, st)
            else:
                y, k = self._rglru(lay, la.mixer, rs, h, meta, st)
            launches += k + 1
            _lib.lm_check(L.ao_lm_streams_update(
                _p(x), _p(y), _lib.DT_F32, n, S, W, _p(hc[2]) if hc else None, _p(hc[1]) if hc else None, dt,
                _p(hn) if taps > 1 else None, _p(rs.canon.x) if taps > 1 else None, taps, _p(meta.slot), _p(meta.back),
                _p(meta.ahead), st), "streams_update")
            # ---- feed-forward sublayer
            if la.ff:
                hc = lay.hc[1]
                _lib.lm_check(L.ao_lm_streams_norm(_p(x), None, n, S, W, _p(hc[0]) if hc else None, _p(lay.norm[1]), dt, 1.0,
                                                   cfg.norm_eps, None, _p(h), st), "streams_norm")
                gu = torch.mm(h, lay.w_gu.t())
                ya = torch.empty(n, la.ff, **act)
                _lib.lm_check(L.ao_lm_gelu_glu(_p(gu), dt, n, la.ff, _p(ya), st), "gelu_glu")
                y = self._mm_f32(ya, lay.w_down)
                _lib.lm_check(L.ao_lm_streams_update(_p(x), _p(y), _lib.DT_F32, n, S, W, _p(hc[2]) if hc else None,
                                                     _p(hc[1]) if hc else None, dt, None, None, 0, None, None, None, st),
                              "streams_update")
                launches += 5
            if after_run is not None:
                after_run(r, x)
        self.launches = launches
        return x

    def _mm_f32(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """a @ w^T with an fp32 result (what fp32 kernels read next)."""
        if a.dtype == torch.bfloat16:
            return torch.mm(a, w.t(), out_dtype=torch.float32)
        return torch.mm(a, w.t())

    def _splits(self, ctas: int, chunk: int) -> int:
        """Key splits of the fp32 attention kernel: enough CTAs to fill the GPU when few rows attend over a long chunk
        (a decoded token late in its chunk).  It depends on sizes only, so a captured graph keeps it."""
        key_blocks = -(-chunk // 32)
        if ctas >= self.sm_count or key_blocks <= 2:
            return 1
        return max(1, min(key_blocks, -(-2 * self.sm_count // ctas), 64))

    def _scan_ws(self, meta: StepMeta, channels: int):
        tf, tc, nt, seg0, segn, ns = meta.scan
        if seg0 is None:
            return None
        nbytes = int(self.L.ao_lm_scan_workspace_bytes(nt, channels))
        return torch.empty(nbytes // 4, dtype=torch.float32, device=self.dev)

    def _parallel(self, lay, mx, rs, h, meta: StepMeta, st):
        """Attention over the chunk + minimal GRU, both from one projection -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        a, Rw, n = mx.left, mx.right_width, meta.n
        H, G, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
        proj = self._mm_f32(h, lay.w_in)                                   # [n][ld] fp32
        qn = torch.empty(n, H, d, dtype=torch.float32, device=dev)
        kn = torch.empty(n, G, d, dtype=tdt, device=dev)
        vn = torch.empty(n, G, dv, dtype=tdt, device=dev)
        both = torch.empty(n, H * dv + Rw, dtype=tdt, device=dev)          # [attention result | recurrence result]
        _lib.lm_check(L.ao_lm_qk_prep(_p(proj), lay.ld, lay.q_off, lay.k_off, lay.v_off, n, H, G, d, dv, self.cfg.norm_eps, dt,
                                      _p(qn), _p(kn), _p(vn), st), "qk_prep")
        tf, tc, nt, tensor = meta.attn[(H, G, d, dv, a.chunk)]
        common = (_p(qn), _p(kn), _p(vn), _p(rs.ring.k), _p(rs.ring.v), dt, proj.data_ptr() + 4 * lay.g_off, lay.ld,
                  _p(lay.dist_bias), lay.dist_bias.shape[1], _p(meta.slot), _p(meta.pos), _p(meta.back), _p(tf), _p(tc), nt, H, G, d,
                  dv, a.chunk, a.scale, a.softcap, mx.left_scale)
        split = 0
        if tensor:
            _lib.lm_check(L.ao_lm_chunk_attention_prompt(*common, _p(both), both.shape[1], st), "chunk_attention_prompt")
        else:
            ns = self._splits(nt * G, a.chunk)
            nbytes = int(L.ao_lm_chunk_attention_workspace_bytes(nt, G, dv, ns))
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
            _lib.lm_check(L.ao_lm_chunk_attention(*common, ns, _p(ws), ws.numel(), _p(both), both.shape[1], st), "chunk_attention")
            split = 1 if ns > 1 else 0
        _lib.lm_check(L.ao_lm_ring_append(_p(kn), _p(vn), n, G * d, G * dv, a.chunk, dt, _p(meta.slot), _p(meta.pos),
                                          _p(meta.ahead), _p(rs.ring.k), _p(rs.ring.v), st), "ring_append")
        sf, sc, snt, seg0, segn, ns = meta.scan
        ws = self._scan_ws(meta, Rw)
        _lib.lm_check(L.ao_lm_mingru_scan(
            _p(proj), lay.ld, lay.z_off, lay.x_off, lay.gr_off, _p(lay.z_b), _p(lay.x_b), dt, Rw, _p(rs.rec.s), _p(meta.slot),
            _p(meta.pos), _p(meta.back), _p(sf), _p(sc), snt, _p(seg0), _p(segn), ns, _p(ws), mx.right_scale,
            both.data_ptr() + H * dv * both.element_size(), both.shape[1], st), "mingru_scan")
        y = self._mm_f32(both, lay.w_out)
        return y, 6 + split + (2 if seg0 is not None else 0)

    def _rglru(self, lay, mx, rs, h, meta: StepMeta, st):
        """gelu branch x real-gated linear recurrence over a short convolution -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        Rw, nb, n = mx.width, mx.blocks, meta.n
        bw = Rw // nb
        proj = self._mm_f32(h, lay.w_in)                                   # [n][y | x] fp32
        u = torch.empty(n, Rw, dtype=torch.float32, device=dev)
        ub = torch.empty(n, Rw, dtype=tdt, device=dev) if tdt != torch.float32 else u
        _lib.lm_check(L.ao_lm_causal_conv(proj.data_ptr() + 4 * Rw, 2 * Rw, _p(lay.x_b), n, Rw, mx.conv, _p(lay.conv_w),
                                          _p(lay.conv_b), dt, 0, _p(rs.conv.x), _p(meta.slot), _p(meta.pos), _p(meta.back),
                                          _p(u), _p(ub) if ub is not u else None, st), "causal_conv")
        ublk = ub.view(n, nb, bw).transpose(0, 1)                          # [blocks][n][bw]
        gates = torch.bmm(ublk, lay.w_gates, out_dtype=torch.float32) if tdt == torch.bfloat16 else torch.bmm(ublk, lay.w_gates)
        out = torch.empty(n, Rw, dtype=tdt, device=dev)
        sf, sc, snt, seg0, segn, ns = meta.scan
        ws = self._scan_ws(meta, Rw)
        _lib.lm_check(L.ao_lm_rglru_scan(
            _p(gates), n, bw, _p(lay.ra_b), _p(lay.ri_b), _p(lay.lam), RGLRU_DECAY, _p(u), _p(proj), 2 * Rw, _p(lay.y_b), dt, Rw,
            _p(rs.rec.s), proj.data_ptr() + 4 * Rw, 2 * Rw, _p(lay.x_b), _p(rs.conv.x) if mx.conv > 1 else None, mx.conv,
            _p(meta.slot), _p(meta.pos),
            _p(meta.back), _p(sf), _p(sc), snt, _p(seg0), _p(segn), ns, _p(ws), _p(out), st), "rglru_scan")
        y = self._mm_f32(out, lay.w_out)
        return y, 5 + (2 if seg0 is not None else 0)

    def _logits(self, x: torch.Tensor, rows: List[int]) -> torch.Tensor:
        """fp32 logits of the given rows: sum of the streams, output norm, head product with an fp32 result."""
        k = len(rows)
        if k == 0:
            return torch.empty(0, self.cfg.vocab_size, dtype=torch.float32, device=self.dev)
        d_rows = torch.tensor(rows, dtype=torch.int32).to(self.dev, non_blocking=True)
        return self._logits_dev(x, d_rows, k)

    def _logits_dev(self, x, d_rows, k, out=None):
        m, cfg, dev = self.m, self.cfg, self.dev
        st = torch.cuda.current_stream(dev).cuda_stream
        xn = torch.empty(k, cfg.width, dtype=m.dtype, device=dev)
        _lib.lm_check(self.L.ao_lm_streams_norm(_p(x), _p(d_rows), k, max(1, cfg.streams), cfg.width, None, _p(m.final_norm),
                                                self.dt, 1.0, cfg.norm_eps, None, _p(xn), st), "streams_norm")
        lg = self._mm_f32(xn, m.head)
        if out is not None:
            out.copy_(lg)
            return out
        return lg

    @torch.no_grad()
    def layer_sums(self, slot: int, tokens) -> Tuple[torch.Tensor, torch.Tensor]:
        """Debugging aid: runs `tokens` as the next tokens of `slot` and returns (logits of all rows, the sum of the
        streams after every layer run [runs][n][W])."""
        st = self.m.states
        t = np.asarray(tokens, np.int64)
        p0 = st.extend(slot, len(t))
        d_tok, meta = self._meta(np.full(len(t), slot, np.int32), np.arange(p0, p0 + len(t), dtype=np.int32), t)
        sums = []
        x = self._layers(d_tok, meta, after_run=lambda r, x: sums.append(x.sum(1)))
        return self._logits(x, list(range(len(t)))), torch.stack(sums)


class GraphDecodeEngine:
    """One decoded token per sequence and step for a fixed batch (slots 0 .. B-1, all at the same position), with the
    tokens, positions and every launch parameter in device memory: the step is captured into a CUDA graph once and
    replayed per token.  Same surface as the Llama DecodeEngine (set_state / step / capture / tok / next_tok / logits)."""

    def __init__(self, model: Tadolix, batch_size: int = 1, temperature: float = 0.8, top_k: Optional[int] = 200):
        assert model.states is not None and model.max_batch_size >= batch_size, "call model.setup_caches first"
        self.model, self.cfg, self.B = model, model.config, batch_size
        self.eng = model.step_engine
        self.device = dev = model.device
        self.temperature, self.top_k = temperature, top_k
        self.S = model.max_seq_length
        B = batch_size
        self.tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.next_tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.logits = torch.zeros(B, self.cfg.vocab_size, dtype=torch.float32, device=dev)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        ones, zeros = torch.ones(B, dtype=torch.int32, device=dev), torch.zeros(B, dtype=torch.int32, device=dev)
        meta = StepMeta()
        meta.n = B
        meta.slot, meta.pos, meta.back, meta.ahead = ar, torch.zeros(B, dtype=torch.int32, device=dev), zeros, zeros
        meta.scan = (ar, ones, B, None, None, 0)       # one row per sequence: every tile is a whole segment
        meta.attn = {shape: (ar, ones, B, False) for shape in self.eng.attn_keys}
        self.meta, self.pos, self.rows = meta, meta.pos, ar
        self.graph = None
        self.graph_stream = None
        self._noise = None
        self._host_pos = 0
        self.launches_per_step = 0
        self.mega = False
        self.tp = None

    def _launch_step(self):
        eng = self.eng
        x = eng._layers(self.tok, self.meta)
        eng._logits_dev(x, self.rows, self.B, out=self.logits)
        self._sample(self.logits)
        self.tok.copy_(self.next_tok)
        self.pos.add_(1)
        self.launches_per_step = eng.launches + 6

    def _sample(self, logits):
        """Greedy: argmax over the fp32 logits.  Otherwise the framework's sampling kernel (temperature, exact top-k,
        exponential-noise argmax), which reads bf16 logits."""
        st = torch.cuda.current_stream(self.device).cuda_stream
        if self.temperature == 0.0:
            _lib.lm_check(self.eng.L.ao_lm_argmax(logits.data_ptr(), logits.stride(0), self.B, logits.shape[1],
                                                  self.next_tok.data_ptr(), st), "argmax")
            return
        if self._noise is None:
            self._noise = torch.empty(logits.shape, dtype=torch.float32, device=self.device)
        noise = self._noise.exponential_(1)
        lb = logits.to(torch.bfloat16)
        _lib.check(_lib.lib().ao_b200_sample(lb.data_ptr(), lb.stride(0), self.B, lb.shape[1], float(self.temperature),
                                             0 if self.top_k is None else int(self.top_k), noise.data_ptr(), noise.stride(0),
                                             self.next_tok.data_ptr(), st), "sample")

    def _state_tensors(self):
        out = []
        for rs in self.model.run_state:
            out += [t for part in (rs.canon, rs.ring, rs.rec, rs.conv) if part is not None for t in part.buffers()]
        return out

    def _with_saved_state(self, fn):
        """Runs fn (trial steps / a capture, which execute the step) and puts tokens, positions and every recurrent
        state of the batch's slots back as they were."""
        tok0, pos0 = self.tok.clone(), self.pos.clone()
        saved = [t[: self.B].clone() for t in self._state_tensors()]
        fn()
        torch.cuda.synchronize(self.device)
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        for t, s in zip(self._state_tensors(), saved):
            t[: self.B].copy_(s)
        torch.cuda.synchronize(self.device)

    def capture(self):
        def trial():
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):   # warm-up outside the capture (library handles, attribute calls)
                    self._launch_step()
            torch.cuda.current_stream(self.device).wait_stream(side)
        self._with_saved_state(trial)

        def cap():
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._launch_step()
        self._with_saved_state(cap)
        return self

    def capture_streaming(self, h_tok, h_out):
        assert h_tok.is_pinned() and h_out.is_pinned() and self.graph is not None

        def cap():
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.tok.copy_(h_tok, non_blocking=True)
                self._launch_step()
                h_out.copy_(self.next_tok, non_blocking=True)
            self.graph_stream = g
        self._with_saved_state(cap)
        return self

    def set_state(self, tokens: torch.Tensor, pos: int):
        """tokens [B] = the token every sequence feeds next, pos = its position (the prompt's length)."""
        if not 0 <= pos < self.S:
            raise ValueError(f"position {pos} outside what setup_caches allowed (max_seq_length {self.S})")
        self.tok.copy_(tokens.reshape(-1).to(torch.int64))
        self.pos.fill_(pos)
        self._host_pos = pos

    def step(self) -> torch.Tensor:
        if self._host_pos >= self.S:
            raise RuntimeError(f"decode step at position {self._host_pos} is past max_seq_length {self.S}")
        self._host_pos += 1
        st = self.model.states
        for b in range(self.B):
            if b in st.length:
                st.length[b] = self._host_pos
        if self.graph is not None:
            self.graph.replay()
        else:
            self._launch_step()
        return self.next_tok

    def check_status(self):
        return None
