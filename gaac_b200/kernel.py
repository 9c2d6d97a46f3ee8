"""Fused decode attention over the compressed KV (head_dim 128, GQA group size 1..8) on the B200 CUDA library.

Mirror of gaac/kernel.py: `attention(q, kp, vp, scale, nsplit)` over two Pages, `choose_nsplit`, and `_ext()` whose
`gaac_attn_launch` keeps the argument list of the reference launcher (gaac/kernel.py:296-300) so callers written against the
reference (its slot cache) work unchanged.  One kernel launch does split-K flash decoding over compressed tiles, the raw BF16
tail and the merge of the splits.
"""
from __future__ import annotations
import functools
import torch
from . import _lib

_WS = {}        # (device index, stream) -> workspace tensor, zeroed once: every call leaves its split counters at zero and the
                # header in front of the partials has a fixed size, so calls of any shape can share it (B*n_q up to 16320)
SM_COUNT_B200 = 148
ATT_WARPS = 16  # warps per CTA of the CUDA kernel (one CTA per SM)


def workspace(dev, B: int, n_q: int, nsplit: int) -> torch.Tensor:
    need = _lib.lib().gaac_attn_workspace_bytes(B, n_q, nsplit)
    key = (torch.device(dev).index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _WS.get(key)
    if ws is None or ws.numel() < need or B * n_q > 16320 or getattr(ws, "_gaac_big", False):
        # a fresh zeroed buffer when none fits, and for the rare shapes whose counters outgrow the fixed-size header
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        ws._gaac_big = B * n_q > 16320
        _WS[key] = ws
    return ws


def workspace_error(dev, B: int = 0, n_q: int = 0) -> bool:
    """True when a kernel that used the cached workspace of the current stream gave up on a bounded wait for its own asynchronous
    copies (the int32 at the start of the workspace).  Reads device memory, so it synchronises; meant for tests and debugging."""
    ws = _WS.get((torch.device(dev).index, torch.cuda.current_stream(dev).cuda_stream))
    return bool(ws is not None and ws[0:4].view(torch.int32).item() != 0)


def choose_nsplit(B: int, n_kv: int, S: int, target_ctas: int = 96, min_tok: int = 512, cap: int = 48) -> int:
    """Splits per (row, kv head), the reference's heuristic verbatim (gaac/kernel.py:340-342; tuned for a 48-SM GB10)."""
    return min(max(1, target_ctas // (B * n_kv)), max(1, S // min_tok), cap)


@functools.lru_cache(maxsize=4096)
def choose_nsplit_sm100(B: int, n_kv: int, S: int, sm_count: int = SM_COUNT_B200, min_tiles_per_warp: int = 2, ragged: bool = False,
                        total_tokens: int | None = None) -> int:
    """Splits per (row, kv head) for a B200.  The kernel runs one 16-warp CTA per SM; a CTA keeps the metadata of the first
    META_TILES (512) tiles of its range in shared memory and fetches the rest from global memory inside the loop.

    Equal lengths (S is every row's length): the split count minimises a cost model fitted to measurements,
        waves x ((tiles per warp + 0.5) x tile time + per-CTA fixed cost),   waves = ceil(rows x splits / SMs),
    over the counts that leave every warp at least min_tiles_per_warp 16-token tiles.  Tile time: 4.5 us for a tile whose
    metadata is staged, 5.2 us beyond; fixed cost (prologue, warp merge, split merge): 10 us.  Few rows end up with one wave that
    fills the SMs, many rows with ranges of at most 512 tiles in several waves.
    Ragged lengths (ragged=True, S is the longest row; total_tokens is accepted and unused): every row gets the same split count;
    see the comment in the code."""
    rows = max(1, B * n_kv)
    ntiles = max(1, (S + 15) // 16)
    most = max(1, ntiles // (ATT_WARPS * min_tiles_per_warp))
    if ragged and B > 1:
        # CTAs are handed out longest row first, so the end of the launch is filled by the small ones and what remains is a
        # trade between the per-CTA fixed cost (grows with the split count) and the last chunks of the longest row (shrink with
        # it): the measured optimum follows sqrt(1.8 x longest row's tiles / rows).  Near it, a count whose CTAs fill whole waves
        # is preferred while the launch is only a few waves long.
        star = (1.8 * ntiles / rows) ** 0.5
        lo, hi = max(1, -(-ntiles // 512)), max(most, 1)
        first = min(max(lo, int(0.6 * star)), hi)
        last = max(first, min(hi, int(1.5 * star) + 1))
        def waste(ns):
            w = rows * ns / sm_count
            return 0.0 if w >= 4 else 1.0 - w / -(-w // 1)
        return min(range(first, last + 1), key=lambda ns: (waste(ns) > 0.1, abs(ns - star)))
    tile_us, tile_far_us, fixed_us, staged = 4.5, 5.2, 10.0, 512
    best, best_t = 1, None
    for ns in range(1, min(most, 2 * sm_count) + 1):
        chunk = -(-ntiles // ns)
        waves = -(-rows * ns // sm_count)
        near, far = min(chunk, staged), max(0, chunk - staged)
        t = waves * (near / ATT_WARPS * tile_us + far / ATT_WARPS * tile_far_us + 0.5 * tile_us + fixed_us)   # tiles are handed out on demand: warps end half a tile apart
        if best_t is None or t < best_t * 0.985:                       # prefer fewer splits unless clearly better
            best, best_t = ns, t
    return best


def _side(sm, codes, flags, tile_off, ovf, head_start, base3, base4, tail) -> _lib.Side:
    return _lib.Side(sm.data_ptr(), codes.data_ptr(), flags.data_ptr(), tile_off.data_ptr(), ovf.data_ptr(), head_start.data_ptr(),
                     ovf.numel(), base3.data_ptr(), base4.data_ptr(), _lib.ptr(tail))


class _Ext:
    """Stand-in for the reference's JIT-built extension module."""

    @staticmethod
    def gaac_attn_launch(smk, ck, fk, tok, ovk, ohsk, b3k, b4k, smv, cv, fv, tov, ovv, ohsv, b3v, b4v,
                         q, slot, n_q, n_kv, SL, S_pad, scale, nsplit, kt, vt, TL, TCAP, out_f32=None, partial=None, exchange=None, fused=False):
        """Same positional arguments as the reference launcher (gaac/kernel.py:296-300): 16 K/V buffers, q [B*n_q, 128] bf16,
        slot int32 [B], n_q, n_kv, SL int32 [heads], S_pad, scale, nsplit, K/V tails [heads, TCAP, 128] bf16 (empty = none),
        TL int32 [heads], TCAP.  Returns out [B*n_q, 128] bf16.  Extras: out_f32 (fp32 tensor to receive the un-rounded
        result), partial ([B*n_q, 130] fp32 tensor: write (m, l, acc) there instead of the output), exchange (a
        gaac_b200._lib.Exchange: push the partial rows into every rank's receive buffer instead and return None; with fused=True
        the same launch also waits for the other ranks' rows, merges them and returns the output)."""
        D = 128
        if q.size(-1) != D:
            raise RuntimeError("head_dim must be 128")
        G = n_q // max(1, n_kv)
        if not (1 <= G <= 8 and G * n_kv == n_q):
            raise RuntimeError("GQA group size must be 1..8")
        if not q.is_cuda:
            raise RuntimeError("gaac_b200 attention needs CUDA tensors: there is no CPU path")
        dev = q.device
        B = slot.size(0)
        has_tail = kt.numel() > 0
        K = _side(smk, ck, fk, tok, ovk, ohsk, b3k, b4k, kt if has_tail else None)
        V = _side(smv, cv, fv, tov, ovv, ohsv, b3v, b4v, vt if has_tail else None)
        ws = workspace(dev, B, n_q, nsplit)
        L = _lib.lib()
        common = (K, V, q.data_ptr(), slot.data_ptr(), B, n_q, n_kv, SL.data_ptr(), S_pad, float(scale), int(nsplit),
                  TL.data_ptr() if has_tail else None, int(TCAP) if has_tail else 0, b3k.size(0), ws.data_ptr(), ws.numel())
        if exchange is not None and fused:
            out = torch.empty(B * n_q, D, dtype=q.dtype, device=dev)
            _lib.check(L.gaac_decode_attn_exchange(*common, exchange, out.data_ptr(), _lib.ptr(out_f32), _lib.stream_ptr(dev)), "gaac_decode_attn_exchange")
            return out
        if exchange is not None:
            _lib.check(L.gaac_decode_attn_push(*common, exchange, _lib.stream_ptr(dev)), "gaac_decode_attn_push")
            return None
        if partial is not None:
            _lib.check(L.gaac_decode_attn_partial(*common, partial.data_ptr(), _lib.stream_ptr(dev)), "gaac_decode_attn_partial")
            return partial
        out = torch.empty(B * n_q, D, dtype=q.dtype, device=dev)
        _lib.check(L.gaac_decode_attn(*common, out.data_ptr(), _lib.ptr(out_f32), _lib.stream_ptr(dev)), "gaac_decode_attn")
        return out


_mod = None


def _ext():
    global _mod
    if _mod is None:
        _lib.lib()          # fail now, loudly, when the library has not been built
        _mod = _Ext()
    return _mod


def attention(q, kp, vp, scale=None, nsplit=None, out_f32=None, out=None):
    """Decode attention over two Pages (kinds 'k' / 'v', H = B*n_kv heads of equal length).
    q: [B, n_q, D] bf16 (one query token per sequence) -> [B, n_q, D] bf16.  (gaac/kernel.py:345-359)
    out (contiguous bf16 tensor of B*n_q*D elements) receives the result instead of a new tensor; out_f32 (fp32, same shape)
    additionally receives the result before its rounding to BF16.
    nsplit=None picks the B200 heuristic; an explicit nsplit is honoured as given.  The two gaac_side descriptors are built
    once and kept on the Page objects, so a decode loop pays one library call per layer."""
    B, n_q, Dq = q.shape
    if Dq != 128:
        raise RuntimeError("head_dim must be 128")
    if not q.is_cuda:
        raise RuntimeError("gaac_b200 attention needs CUDA tensors: there is no CPU path")
    n_kv = kp.H // B
    G = n_q // max(1, n_kv)
    if not (1 <= G <= 8 and G * n_kv == n_q):
        raise RuntimeError("GQA group size must be 1..8")
    dev = q.device
    if nsplit is None: nsplit = choose_nsplit_sm100(B, n_kv, kp.S)
    if out is None:
        out = torch.empty(B * n_q, Dq, dtype=q.dtype, device=dev)
    elif not (out.is_contiguous() and out.dtype == q.dtype and out.numel() == B * n_q * Dq):
        raise RuntimeError("out must be a contiguous bf16 tensor with B*n_q*128 elements")
    _pages_call(q, kp, vp, B, n_q, n_kv, scale, nsplit, out=out, out_f32=out_f32)
    return out.view(B, n_q, Dq)


def _page_side(pg) -> _lib.Side:
    """The gaac_side descriptor of a Page, built once and kept on the Page object (rebuilt when its escape stream was replaced)."""
    sd = getattr(pg, "_attn_side", None)
    if pg.S == 0:                                  # a Page without tokens (a rank past the end of a short context): nothing is read through
        if sd is None:                             # these pointers, but the library wants them non-null, so they point at a small zero buffer
            z = torch.zeros(256, dtype=torch.uint8, device=pg.base3.device)
            sd = _side(z, z, z, z, z, pg.ovf_head_start, pg.base3, pg.base4, None)
            pg._attn_side, pg._attn_keep = sd, z
        return sd
    if sd is None or sd.ovf != pg.ovf.data_ptr() or sd.sm != pg.sm.data_ptr():
        sd = _side(pg.sm, pg.codes, pg.flags, pg.tile_off, pg.ovf, pg.ovf_head_start, pg.base3, pg.base4, None)
        pg._attn_side = sd
    return sd


def _pages_call(q, kp, vp, B, n_q, n_kv, scale, nsplit, out=None, out_f32=None, part=None, exchange=None, fused=False):
    """One gaac_decode_attn_pages call: every head of the two Pages holds kp.S tokens and batch row b reads heads b*n_kv ..,
    which is all the identity slot map and the constant length table of the reference's entry point said
    (gaac/kernel.py:349-352); the kernel needs neither table."""
    dev = q.device
    q2 = q.reshape(B * n_q, 128)
    if not q2.is_contiguous(): q2 = q2.contiguous()
    ws = workspace(dev, B, n_q, nsplit)
    _lib.check(_lib.lib().gaac_decode_attn_pages(_page_side(kp), _page_side(vp), q2.data_ptr(), B, n_q, n_kv, kp.S, max(16, kp.sm.shape[1] // 128),
                                                 float(scale if scale is not None else 128 ** -0.5), int(nsplit), kp.base3.size(0),
                                                 ws.data_ptr(), ws.numel(), _lib.ptr(out), _lib.ptr(out_f32), _lib.ptr(part), exchange,
                                                 1 if fused else 0, _lib.stream_ptr(dev)), "gaac_decode_attn_pages")


def combine(pm: torch.Tensor, pl: torch.Tensor, pa: torch.Tensor, out_f32: torch.Tensor | None = None) -> torch.Tensor:
    """Merge partials pm, pl [n_heads, n_parts] and pa [n_heads, n_parts, 128] (fp32, m in natural-log units) -> [n_heads, 128] bf16
    (gaac/kernel.py:281-294)."""
    n_heads, n_parts = pm.shape
    out = torch.empty(n_heads, 128, dtype=torch.bfloat16, device=pm.device)
    _lib.check(_lib.lib().gaac_combine(pm.contiguous().data_ptr(), pl.contiguous().data_ptr(), pa.contiguous().data_ptr(), n_heads, n_parts,
                                       out.data_ptr(), _lib.ptr(out_f32), _lib.stream_ptr(pm.device)), "gaac_combine")
    return out


def combine_parts(parts: torch.Tensor, out_f32: torch.Tensor | None = None) -> torch.Tensor:
    """Merge packed partials [n_parts, n_heads, 130] fp32 (rows of (m, l, acc[128]), m in natural-log units) -> [n_heads, 128] bf16:
    the buffer an all-gather of the ranks' partial outputs produces, merged in one launch."""
    n_parts, n_heads, w = parts.shape
    assert w == 130 and parts.is_contiguous()
    out = torch.empty(n_heads, 128, dtype=torch.bfloat16, device=parts.device)
    _lib.check(_lib.lib().gaac_combine_parts(parts.data_ptr(), n_heads, n_parts, out.data_ptr(), _lib.ptr(out_f32), _lib.stream_ptr(parts.device)),
               "gaac_combine_parts")
    return out
