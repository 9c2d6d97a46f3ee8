"""CPU oracle for the GAAC KV codec and compressed-KV decode attention (numpy).

TEST INFRASTRUCTURE ONLY.  This module is the checker used by the test-suite, by the smoke test and by the
CPU-baseline leg of the benchmark.  Nothing in the product package imports it; the product path is the CUDA
library and fails loudly when that library is missing.

Every function restates, in plain numpy, the algorithm of one function of the reference implementation
(Intelligent-Microsystems-Lab/GAAC) and cites the reference file:line it follows.  Parity pin: the restatement
is checked against outputs of the reference itself (its torch codec run on CPU and its Triton kernels run under the
Triton interpreter); those outputs are committed as fixtures under tests/golden/ together with the script that
produced them.

Conventions: BF16 tensors are carried as uint16 bit patterns; "kind" is 'k' or 'v'.
"""
from __future__ import annotations
import numpy as np

D = 128          # head dim                       gaac/codec.py:23
T = 16           # tokens per tile                gaac/codec.py:24
GS = 8           # elements per group             gaac/codec.py:25
CB = D * 3 // 8  # code bytes per token row       gaac/codec.py:26
NG = D // GS
TILE_MAX_ESC = 1280     # gaac/kv_cache.py:19
SM_OFF, CD_OFF, FL_OFF, OVF_OFF = 0, 2048, 2816, 2880   # paged tile slot layout, gaac/vllm/store.py:18


# --------------------------------------------------------------------------------------------- permutations
def perm_k() -> np.ndarray:
    """Stored position -> channel for K (gaac/codec.py:29-36): position 32j+4s+q = channel 16s+2j+{0,1,8,9}[q]."""
    p = np.empty(D, dtype=np.int64)
    for j in range(4):
        for s in range(8):
            for q, off in enumerate((0, 1, 8, 9)):
                p[32 * j + 4 * s + q] = 16 * s + 2 * j + off
    return p


def perm_v() -> np.ndarray:
    """Stored position -> channel for V (gaac/codec.py:39-45): position 16r+n = channel 8n+r."""
    p = np.empty(D, dtype=np.int64)
    for r in range(8):
        for n in range(16):
            p[16 * r + n] = 8 * n + r
    return p


def perm(kind: str) -> np.ndarray:
    return perm_k() if kind == "k" else perm_v()


def storage_index(kind: str) -> tuple[np.ndarray, np.ndarray]:
    """(sm_idx[T*D], code_idx[T*CB]): storage byte -> token-major byte inside one tile (gaac/codec.py:52-67)."""
    sm_idx, cd_idx = [], []
    if kind == "k":
        for o in range(T // 8):
            for l in range(32):
                tok, j = 8 * o + (l >> 2), l & 3
                sm_idx += [tok * D + 32 * j + q for q in range(32)]
                cd_idx += [tok * CB + 12 * j + q for q in range(12)]
    else:
        for l in range(32):
            j, r = l & 3, l >> 2
            for tok in (2 * j, 2 * j + 1, 2 * j + 8, 2 * j + 9):
                sm_idx += [tok * D + 16 * r + q for q in range(16)]
                cd_idx += [tok * CB + 6 * r + q for q in range(6)]
    return np.asarray(sm_idx, dtype=np.int64), np.asarray(cd_idx, dtype=np.int64)


# --------------------------------------------------------------------------------------------- calibration
def exponent_hist(x16: np.ndarray, n_kv: int) -> np.ndarray:
    """x16: [..., n_kv, D] uint16 (token-major) -> int64 [n_kv*D, 256] exponent histogram (gaac/codec.py:80-84)."""
    e = ((x16.astype(np.int64) >> 7) & 0xFF).reshape(-1, n_kv * D)
    hist = np.zeros((n_kv * D, 256), dtype=np.int64)
    cols = np.arange(n_kv * D)
    for row in e:
        np.add.at(hist, (cols, row), 1)
    return hist


def exponent_hist_fast(x16: np.ndarray, n_kv: int) -> np.ndarray:
    """Same result as exponent_hist with one bincount (the form the reference uses, gaac/codec.py:82-84)."""
    e = ((x16.astype(np.int64) >> 7) & 0xFF).reshape(-1, n_kv * D)
    idx = np.arange(n_kv * D, dtype=np.int64)[None, :] * 256 + e
    return np.bincount(idx.reshape(-1), minlength=n_kv * D * 256).reshape(n_kv * D, 256)


def bases_from_hist(hist: np.ndarray, n_kv: int) -> tuple[np.ndarray, np.ndarray]:
    """Start of the densest 8-wide / 16-wide exponent window, first maximum wins (gaac/codec.py:70-77)."""
    cs = np.concatenate([np.zeros((hist.shape[0], 1), dtype=np.int64), np.cumsum(hist.astype(np.int64), 1)], 1)
    out = []
    for w in (8, 16):
        out.append(np.argmax(cs[:, w:] - cs[:, :-w], 1).astype(np.uint8).reshape(n_kv, D))
    return out[0], out[1]


def calibrate(sample16: np.ndarray, n_kv: int) -> tuple[np.ndarray, np.ndarray]:
    """sample16: [H, Tn, D] uint16, head h uses bases of h % n_kv (gaac/codec.py:121-126)."""
    H = sample16.shape[0]
    x = sample16.reshape(H // n_kv, n_kv, -1, D).transpose(0, 2, 1, 3)
    return bases_from_hist(exponent_hist_fast(np.ascontiguousarray(x), n_kv), n_kv)


# --------------------------------------------------------------------------------------------- encoder
def _tiers_codes(x16p: np.ndarray, b3p: np.ndarray, b4p: np.ndarray):
    """x16p: [..., D] int64 bit patterns in stored order; b3p/b4p broadcastable int64 bases in stored order.
    Returns (sm, e, d4, tier[..., NG], code[..., D]) following gaac/codec.py:139-150."""
    e = (x16p >> 7) & 0xFF
    sm = ((x16p >> 8) & 0x80) | (x16p & 0x7F)
    d3, d4 = e - b3p, e - b4p
    shp = x16p.shape[:-1]
    g3 = ((d3 >= 0) & (d3 < 8)).reshape(*shp, NG, GS).all(-1)
    g4 = ((d4 >= 0) & (d4 < 16)).reshape(*shp, NG, GS).all(-1)
    tier = np.where(g3, 0, np.where(g4, 1, 2)).astype(np.int64)
    tier_e = np.repeat(tier, GS, axis=-1)
    code = np.where(tier_e == 0, d3 & 7, np.where(tier_e == 1, d4 & 7, e & 7))
    return sm, e, d4, tier, code


def _pack_codes(code: np.ndarray) -> np.ndarray:
    """[..., D] 3-bit codes -> [..., CB] bytes: bit k of code i at bit 3i+k of a little-endian string (codec.py:151-152)."""
    bits = ((code[..., None] >> np.arange(3)) & 1).astype(np.uint8).reshape(*code.shape[:-1], D * 3)
    return np.packbits(bits, axis=-1, bitorder="little")


def _escape_bytes(e: np.ndarray, d4: np.ndarray, tier: np.ndarray):
    """Per group escape bytes (gaac/codec.py:155-172): tier 1 -> 1 byte (bit i = 4th bit of d4_i), tier 2 -> 5 bytes
    (40-bit LE of the eight 5-bit fields e_i >> 3).  Returns (bytes [..., NG, 5] uint8, size [..., NG])."""
    shp = tier.shape[:-1]
    eg = e.reshape(*shp, NG, GS)
    d4g = d4.reshape(*shp, NG, GS)
    bit4 = (((d4g >> 3) & 1) << np.arange(GS)).sum(-1)
    w40 = ((eg >> 3) << (5 * np.arange(GS))).sum(-1)
    raw5 = (w40[..., None] >> (8 * np.arange(5))) & 0xFF
    by = np.where((tier == 2)[..., None], raw5, 0)
    by[..., 0] = np.where(tier == 1, bit4, by[..., 0])
    size = np.where(tier == 1, 1, np.where(tier == 2, 5, 0))
    return by.astype(np.uint8), size.astype(np.int64)


def encode(x16: np.ndarray, base3: np.ndarray, base4: np.ndarray, kind: str, n_kv: int, bidx: np.ndarray | None = None) -> dict:
    """Reference encoder (gaac/codec.py:133-184).  x16: [H, S, D] uint16; base3/base4: uint8 [rows, D]; head h uses base
    row h % n_kv, or bidx[h] when given (gaac/encoder.py:21-24).  Returns the Page fields as numpy arrays."""
    H, S, _ = x16.shape
    p = perm(kind)
    xp = x16.astype(np.int64)[..., p]
    rows = (np.arange(H) % n_kv) if bidx is None else np.asarray(bidx, dtype=np.int64)
    b3p = base3.astype(np.int64)[rows][:, p][:, None, :]
    b4p = base4.astype(np.int64)[rows][:, p][:, None, :]
    sm, e, d4, tier, code = _tiers_codes(xp, b3p, b4p)
    codes_tok = _pack_codes(code)
    g = np.arange(NG)
    flags = (((tier >= 1).astype(np.int64) << (2 * g)) | ((tier == 2).astype(np.int64) << (2 * g + 1))).sum(-1)
    esc, gsize = _escape_bytes(e, d4, tier)
    row_bytes = gsize.sum(-1)
    head_start = np.concatenate([[0], np.cumsum(row_bytes.sum(-1))]).astype(np.int64)
    ovf_off = np.cumsum(row_bytes, 1) - row_bytes
    total = int(head_start[-1])
    keep = np.arange(5)[None, None, None, :] < gsize[..., None]
    ovf = np.concatenate([esc[keep], np.zeros(8, dtype=np.uint8)])      # +8: readers may fetch a whole 5-byte group at the end
    assert ovf.size == total + 8
    S_pad = (S + T - 1) // T * T
    smu = sm.astype(np.uint8)
    if S_pad != S:
        smu = np.concatenate([smu, np.zeros((H, S_pad - S, D), dtype=np.uint8)], 1)
        codes_tok = np.concatenate([codes_tok, np.zeros((H, S_pad - S, CB), dtype=np.uint8)], 1)
    si, ci = storage_index(kind)
    sm_st = smu.reshape(H, S_pad // T, T * D)[:, :, si].reshape(H, S_pad * D)
    cd_st = codes_tok.reshape(H, S_pad // T, T * CB)[:, :, ci].reshape(H, S_pad * CB)
    flags32 = np.zeros((H, S_pad), dtype=np.int64)
    flags32[:, :S] = flags
    return dict(sm=np.ascontiguousarray(sm_st), codes=np.ascontiguousarray(cd_st),
                flags=flags32.astype(np.uint32).view(np.int32), ovf_off=ovf_off.astype(np.int32), ovf=ovf,
                ovf_head_start=head_start.astype(np.int32), tile_off=np.ascontiguousarray(ovf_off[:, ::T]).astype(np.int32),
                base3=base3, base4=base4, H=H, S=S, n_kv=n_kv, kind=kind, tile_bytes=_tile_bytes(row_bytes, S_pad))


def _tile_bytes(row_bytes: np.ndarray, S_pad: int) -> np.ndarray:
    H, S = row_bytes.shape
    rb = np.zeros((H, S_pad), dtype=np.int64)
    rb[:, :S] = row_bytes
    return rb.reshape(H, S_pad // T, T).sum(-1).astype(np.int32)


def row_offsets(flags: np.ndarray, S: int) -> np.ndarray:
    """Row offsets within each head's escape stream from the tag words (gaac/codec.py:221-225)."""
    f = flags[:, :S].astype(np.int64) & 0xFFFFFFFF
    rb = sum(((f >> (2 * g)) & 1) + 4 * ((f >> (2 * g + 1)) & 1) for g in range(NG))
    return (np.cumsum(rb, 1) - rb).astype(np.int32)


# --------------------------------------------------------------------------------------------- decoder
def decode_rows(sm: np.ndarray, cd: np.ndarray, flags: np.ndarray, esc_at, b3p: np.ndarray, b4p: np.ndarray) -> np.ndarray:
    """Token-major rows -> uint16 values in stored order (gaac/codec.py:196-215).
    sm [..., D], cd [..., CB] int64, flags [...] int64, esc_at(gstart_offsets[..., NG], k) -> escape byte k of a group."""
    bits = np.unpackbits(cd.astype(np.uint8), axis=-1, bitorder="little").reshape(*cd.shape[:-1], D, 3).astype(np.int64)
    code = bits[..., 0] | (bits[..., 1] << 1) | (bits[..., 2] << 2)
    f = flags.astype(np.int64) & 0xFFFFFFFF
    tier = np.stack([(f >> (2 * g)) & 3 for g in range(NG)], -1)       # 0, 1, 3
    gsize = np.where(tier == 1, 1, np.where(tier == 3, 5, 0))
    gstart = np.cumsum(gsize, -1) - gsize
    by = np.stack([esc_at(gstart, k) for k in range(5)], -1).astype(np.int64)
    bit4 = ((by[..., 0][..., None] >> np.arange(GS)) & 1).reshape(*sm.shape)
    w40 = (by << (8 * np.arange(5))).sum(-1)
    hi5 = ((w40[..., None] >> (5 * np.arange(GS))) & 31).reshape(*sm.shape)
    tier_e = np.repeat(tier, GS, axis=-1)
    exp = np.where(tier_e == 0, b3p + code, np.where(tier_e == 1, b4p + (code | (bit4 << 3)), code | (hi5 << 3)))
    return ((sm & 0x80) << 8) | (exp << 7) | (sm & 0x7F)


def decode(page: dict) -> np.ndarray:
    """Bit-exact reconstruction of a Page -> [H, S, D] uint16 (gaac/codec.py:186-218)."""
    H, S, kind, n_kv = page["H"], page["S"], page["kind"], page["n_kv"]
    S_pad = page["sm"].shape[1] // D
    si, ci = storage_index(kind)
    inv_s = np.empty_like(si); inv_s[si] = np.arange(si.size)
    inv_c = np.empty_like(ci); inv_c[ci] = np.arange(ci.size)
    sm = page["sm"].reshape(H, S_pad // T, T * D)[:, :, inv_s].reshape(H, S_pad, D)[:, :S].astype(np.int64)
    cd = page["codes"].reshape(H, S_pad // T, T * CB)[:, :, inv_c].reshape(H, S_pad, CB)[:, :S].astype(np.int64)
    p = perm(kind)
    rows = np.asarray(page.get("bidx")) if page.get("bidx") is not None else np.arange(H) % n_kv
    b3p = page["base3"].astype(np.int64)[rows][:, p][:, None, :]
    b4p = page["base4"].astype(np.int64)[rows][:, p][:, None, :]
    ovf = page["ovf"].astype(np.int64)
    base = page["ovf_head_start"][:-1].astype(np.int64).reshape(H, 1, 1) + page["ovf_off"].astype(np.int64)[..., None]

    def esc_at(gstart, k):
        return ovf[np.minimum(base + gstart + k, ovf.size - 1)]

    raw16 = decode_rows(sm, cd, page["flags"][:, :S], esc_at, b3p, b4p)
    out = np.empty((H, S, D), dtype=np.int64)
    out[..., p] = raw16
    return out.astype(np.uint16)


# --------------------------------------------------------------------------------------------- attention
def bf16_to_f64(x16: np.ndarray) -> np.ndarray:
    return (x16.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def attention_ref(q16: np.ndarray, k16: np.ndarray, v16: np.ndarray, scale: float, with_abs: bool = False):
    """q16 [n_q, D], k16/v16 [L, n_kv, D] uint16 -> [n_q, D] float64.  GQA: q head j uses kv head j // G
    (tests/common.py:15-22, computed in float64 here).  L == 0 gives zeros (gaac/kernel.py:293).
    with_abs=True returns (out, out_abs) with out_abs = sum_i p_i |v_i|, the magnitude that a relative error of the softmax
    weights is multiplied by (see attention_bound)."""
    n_q, n_kv = q16.shape[0], k16.shape[1]
    G = n_q // n_kv
    if k16.shape[0] == 0:
        z = np.zeros((n_q, D))
        return (z, z.copy()) if with_abs else z
    q = bf16_to_f64(q16)
    k = np.repeat(bf16_to_f64(k16), G, axis=1).transpose(1, 0, 2)      # [n_q, L, D]
    v = np.repeat(bf16_to_f64(v16), G, axis=1).transpose(1, 0, 2)
    s = np.einsum("hld,hd->hl", k, q) * scale
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    out = np.einsum("hl,hld->hd", p, v)
    if with_abs:
        return out, np.einsum("hl,hld->hd", p, np.abs(v))
    return out


ATTN_TOL = 2e-3              # max-abs bound on the fp32 attention result at unit scale
WEIGHT_REL_ERR = 2.0 ** -12  # bound on the relative error of one softmax weight as the kernels under test compute it


def attention_bound(out_abs: np.ndarray) -> np.ndarray:
    """Per-element bound on |fp32 result - float64 reference|: 2e-3 wherever the weighted magnitude sum_i p_i |v_i| (out_abs from
    attention_ref) is at most 8.2, and 2^-12 times that magnitude above it.  Where the 2^-12 comes from: a score is a sum of 128
    BF16 products accumulated in fp32 (absolute error of a few 1e-5 in the exponent at the magnitudes of the test data), and the
    weight enters the PV product as a pair of BF16 numbers (relative error 2^-16); the bound leaves a factor of several on both.
    A kernel that feeds the weights as single BF16 numbers, as the reference's does (gaac/kernel.py:178), has 2^-8 per weight and
    would need 16 times this bound."""
    return np.maximum(ATTN_TOL, WEIGHT_REL_ERR * out_abs)


def combine_partials(pm: np.ndarray, pl: np.ndarray, pa: np.ndarray) -> np.ndarray:
    """Merge split partials (gaac/kernel.py:281-294): pm, pl [..., NS], pa [..., NS, D] -> [..., D] float64.
    M = max m; L = sum l*exp(m-M) over finite m; O = sum acc*exp(m-M) / L, 0 when L <= 0."""
    pm = pm.astype(np.float64); pl = pl.astype(np.float64); pa = pa.astype(np.float64)
    M = pm.max(-1, keepdims=True)
    with np.errstate(invalid="ignore"):
        f = np.where(np.isneginf(pm), 0.0, np.exp(pm - M))
    L = (pl * f).sum(-1)
    A = (pa * f[..., None]).sum(-2)
    with np.errstate(invalid="ignore", divide="ignore"):
        return np.where(L[..., None] > 0, A / L[..., None], 0.0)


def choose_nsplit(B: int, n_kv: int, S: int, target_ctas: int = 96, min_tok: int = 512, cap: int = 48) -> int:
    """gaac/kernel.py:340-342."""
    return min(max(1, target_ctas // (B * n_kv)), max(1, S // min_tok), cap)


# --------------------------------------------------------------------------------------------- page accounting
def page_nbytes(page: dict) -> int:
    """Stored bytes of a Page (gaac/codec.py:104-108)."""
    esc = int(page["ovf_head_start"][-1]) - int(page["ovf_head_start"][0])
    return page["H"] * page["S"] * (D + CB + 4) + esc + page["H"] * ((page["S"] + T - 1) // T) * 4


def page_ratio(page: dict) -> float:
    return page["H"] * page["S"] * D * 2 / page_nbytes(page)


# --------------------------------------------------------------------------------------------- slot cache model (layout A)
class SlotCacheModel:
    """Behavioural model of gaac/kv_cache.py CompressedKVCache for one kind: per cache head a list of finalized
    16-token tiles (encoded) plus a raw tail.  State after prefill/append is expressed as the buffers of
    _Store (gaac/kv_cache.py:99-119) so a device implementation can be compared byte for byte."""

    def __init__(self, kind: str, H: int, cap: int, ovf_cap: int, base3: np.ndarray, base4: np.ndarray):
        self.kind, self.H, self.cap, self.ovf_cap = kind, H, cap, ovf_cap
        self.sm = np.zeros((H, cap * D), np.uint8)
        self.codes = np.zeros((H, cap * CB), np.uint8)
        self.flags = np.zeros((H, cap), np.int32)
        self.tile_off = np.zeros((H, cap // T), np.int32)
        self.ovf = np.zeros(H * ovf_cap, np.uint8)
        self.ovf_used = np.zeros(H, np.int32)
        self.tail = np.zeros((H, T, D), np.uint16)
        self.base3, self.base4 = base3, base4
        self.S = np.zeros(H, np.int32)
        self.tail_len = np.zeros(H, np.int32)

    def _put_tile(self, h: int, tile: int, rows16: np.ndarray):
        """Encode one full tile of head h in place and append its escapes (gaac/kv_cache.py:30-68)."""
        nb = self.base3.shape[0]
        pg = encode(rows16[None], self.base3, self.base4, self.kind, nb, bidx=np.array([h % nb]))
        self.sm[h, tile * T * D:(tile + 1) * T * D] = pg["sm"][0]
        self.codes[h, tile * T * CB:(tile + 1) * T * CB] = pg["codes"][0]
        self.flags[h, tile * T:(tile + 1) * T] = pg["flags"][0]
        n = int(pg["ovf_head_start"][-1]); used = int(self.ovf_used[h])
        self.ovf[h * self.ovf_cap + used: h * self.ovf_cap + used + n] = pg["ovf"][:n]
        self.tile_off[h, tile] = used
        self.ovf_used[h] = used + n

    def prefill(self, h0: int, x16: np.ndarray):
        """x16: [n_heads, L, D] for cache heads h0.. (gaac/kv_cache.py:149-169)."""
        n, L, _ = x16.shape
        Sf = L // T * T
        for i in range(n):
            h = h0 + i
            self.ovf_used[h] = 0
            for t in range(Sf // T):
                self._put_tile(h, t, x16[i, t * T:(t + 1) * T])
            if L > Sf:
                self.tail[h, :L - Sf] = x16[i, Sf:]
            self.S[h] = Sf; self.tail_len[h] = L - Sf

    def append(self, h: int, row16: np.ndarray):
        """One new token for cache head h (gaac/kv_cache.py:22-29,87-96)."""
        pos = int(self.tail_len[h])
        self.tail[h, pos] = row16
        if pos + 1 == T:
            self._put_tile(h, int(self.S[h]) // T, self.tail[h])
            self.tail_len[h] = 0; self.S[h] += T
        else:
            self.tail_len[h] = pos + 1


# --------------------------------------------------------------------------------------------- paged store model (layout B)
class PagedStoreModel:
    """Behavioural model of gaac/vllm/store.py (one layer).  Physical tile p = block*(2*n_kv) + 2*kvh + kind_index;
    mt[p] == p: compressed in its slot of `buf`; mt[p] == ~r: raw bf16 tile r of the side pool.  The order in which
    concurrent programs pop raw tiles is unspecified in the reference (atomic), so callers compare decoded content
    and the free-tile count, not raw tile numbers."""

    def __init__(self, num_blocks: int, n_kv: int, raw_tiles: int, bases: dict, ovf_slot: int):
        self.n_kv, self.ovf_slot, self.TS = n_kv, ovf_slot, OVF_OFF + ovf_slot
        self.mt = np.arange(num_blocks * 2 * n_kv, dtype=np.int64)
        self.raw = np.zeros((raw_tiles, T, D), np.uint16)
        self.stack = list(range(raw_tiles))          # top of stack = end of list
        self.err = 0
        self.bases = bases
        self.buf = np.zeros(num_blocks * 2 * n_kv * self.TS, np.uint8)

    def _pop(self):
        if not self.stack:
            self.err += 1
            return None
        return self.stack.pop()

    def store(self, key16: np.ndarray, value16: np.ndarray, ent: np.ndarray):
        """key16/value16: [num_tokens, n_kv, D]; ent: [E, 4] = (blk, tok0, off0, n) (gaac/vllm/store.py:22-105)."""
        freed = []
        for blk, tok0, off0, n in ent.tolist():
            if blk < 0:
                continue
            for t in range(2 * self.n_kv):
                kind, kvh = ("k", "v")[t & 1], t >> 1
                src = key16 if kind == "k" else value16
                p = blk * 2 * self.n_kv + t
                old = int(self.mt[p]); have = old < 0
                r_old = -old - 1 if have else None
                rows = np.zeros((T, D), np.uint16)
                if have and off0 > 0:
                    rows[:off0] = self.raw[r_old, :off0]
                rows[off0:off0 + n] = src[tok0:tok0 + n, kvh]
                if off0 + n == T:
                    b3, b4 = self.bases[kind + "3"], self.bases[kind + "4"]
                    pg = encode(rows[None], b3, b4, kind, b3.shape[0], bidx=np.array([kvh]))
                    total = int(pg["ovf_head_start"][-1])
                    if total <= self.ovf_slot:
                        base = p * self.TS
                        self.buf[base + SM_OFF: base + SM_OFF + T * D] = pg["sm"][0]
                        self.buf[base + CD_OFF: base + CD_OFF + T * CB] = pg["codes"][0]
                        self.buf[base + FL_OFF: base + FL_OFF + 64] = pg["flags"][0].view(np.uint8)
                        self.buf[base + OVF_OFF: base + OVF_OFF + total] = pg["ovf"][:total]
                        self.mt[p] = p
                        if have:
                            freed.append(r_old)
                        continue
                    need_pop = not have
                else:
                    need_pop = not have
                r = r_old if have else (self._pop() if need_pop else None)
                if r is None:
                    r = 0       # failed pop: the reference writes to tile 0 and counts the error (store.py:68-70,97-99)
                self.raw[r, off0:off0 + n] = src[tok0:tok0 + n, kvh]
                self.mt[p] = -r - 1
        for r in freed:          # _free_tiles (gaac/vllm/store.py:108-114)
            self.stack.append(r)

    def release_blocks(self, blocks):
        """gaac/vllm/store.py:166-174."""
        for blk in blocks:
            for t in range(2 * self.n_kv):
                p = blk * 2 * self.n_kv + t
                if self.mt[p] < 0:
                    self.stack.append(int(-self.mt[p] - 1)); self.mt[p] = p

    def decode_tile(self, blk: int, kvh: int, kind: str) -> np.ndarray:
        """One tile -> [16, D] uint16 in natural channel order (gaac/vllm/store.py:117-163)."""
        t = 2 * kvh + (0 if kind == "k" else 1)
        p = blk * 2 * self.n_kv + t
        m = int(self.mt[p])
        if m < 0:
            return self.raw[-m - 1].copy()
        base = p * self.TS
        b3, b4 = self.bases[kind + "3"], self.bases[kind + "4"]
        page = dict(sm=self.buf[base + SM_OFF: base + SM_OFF + T * D][None].copy(),
                    codes=self.buf[base + CD_OFF: base + CD_OFF + T * CB][None].copy(),
                    flags=self.buf[base + FL_OFF: base + FL_OFF + 64].copy().view(np.int32)[None],
                    ovf=np.concatenate([self.buf[base + OVF_OFF: base + self.TS], np.zeros(8, np.uint8)]),
                    ovf_head_start=np.array([0, self.ovf_slot], np.int32), base3=b3, base4=b4,
                    H=1, S=T, n_kv=b3.shape[0], kind=kind, bidx=np.array([kvh]))
        page["ovf_off"] = row_offsets(page["flags"], T)
        return decode(page)[0]


# --------------------------------------------------------------------------------------------- synthetic workloads
def synth_kv(kind: str, H: int, S: int, seed: int, raw_frac: float = 0.002, four_frac: float = 0.10) -> np.ndarray:
    """Seeded synthetic KV of the benchmark configurations -> [H, S, D] uint16 (BF16 bits).

    x[h,t,d] = N(0,1) * s[h,d] with s = exp(N(0, 1.0)) for K and exp(N(0, 0.5)) for V (drawn per (head, channel)),
    rounded to BF16.  Per (head, token, stored group of 8): with probability raw_frac one element is multiplied by 2^7
    (forces the raw tier), with probability four_frac one element by 2^4 (forces the 4-bit window)."""
    rng = np.random.default_rng([seed, 0 if kind == "k" else 1])
    sd = 1.0 if kind == "k" else 0.5
    s = np.exp(rng.standard_normal((H, 1, D), dtype=np.float32) * sd)
    out = np.empty((H, S, D), dtype=np.uint16)
    p = perm(kind)
    inv = np.empty_like(p); inv[p] = np.arange(D)
    step = 8192
    for t0 in range(0, S, step):
        n = min(step, S - t0)
        x = rng.standard_normal((H, n, D), dtype=np.float32) * s
        xs = x[..., p].reshape(H, n, NG, GS)
        u = rng.random((H, n, NG), dtype=np.float32)
        pos = rng.integers(0, GS, (H, n, NG))
        mult = np.where(u < raw_frac, 128.0, np.where(u < raw_frac + four_frac, 16.0, 1.0)).astype(np.float32)
        onehot = pos[..., None] == np.arange(GS)
        xs = np.where(onehot, xs * mult[..., None], xs)
        out[:, t0:t0 + n] = f32_to_bf16(xs.reshape(H, n, D)[..., inv])
    return out


def kv_like(H: int, S: int, seed: int, outliers: float = 1e-3) -> np.ndarray:
    """Fixture in the style of the reference tests (tests/common.py:4-12): Gaussian x per-channel scale 2^(U*8-4)
    shared across heads, 0.1 % of elements x 1e4 -> [H, S, D] uint16.  (Own seeded stream, not torch's.)"""
    rng = np.random.default_rng([seed, 77])
    scale = np.exp2(rng.random((1, 1, D), dtype=np.float32) * 8 - 4)
    x = rng.standard_normal((H, S, D), dtype=np.float32) * scale
    m = rng.random((H, S, D), dtype=np.float32) < outliers
    return f32_to_bf16(np.where(m, x * 1e4, x))


def tier_shares(flags: np.ndarray, S: int) -> tuple[float, float, float]:
    f = flags[:, :S].astype(np.int64) & 0xFFFFFFFF
    t = np.stack([(f >> (2 * g)) & 3 for g in range(NG)], -1)
    n = t.size
    return float((t == 0).sum() / n), float((t == 1).sum() / n), float((t == 3).sum() / n)
