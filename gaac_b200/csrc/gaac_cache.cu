// Cache maintenance kernels (sm_100a): slot-layout append, paged-layout store / release / block decode.
#include "gaac_api.cuh"
#include "gaac_warp.cuh"

namespace gaac {

// ------------------------------------------------------------------------------------------------ slot layout: append
struct AppendParams {
  gaac_store K, V;
  const uint16_t *k_new, *v_new;
  const int* slot; int n_kv;
  int *tail_len, *seq_len;
  long S_cap, ovf_cap; int n_base_rows;
  int* err;
};

// One CTA per (batch row, kv head): warp 0 appends K, warp 1 appends V; the shared counters are advanced once both are done
// (the reference needs a second launch for that: gaac/kv_cache.py:72-73,87-96).
// First half: the new row goes into the tail; when that fills the tail, the 16 rows are encoded into registers.  Returns the
// tile's escape bytes, or -1 when there is no tile to store (tail not full, or the head is at its token capacity).
template <int KIND_V>
__device__ __forceinline__ int append_encode(WarpScratch& ws, const gaac_store& st, const uint16_t* xrow, long h, int pos, int tile, long S_cap,
                                             int n_base_rows, int lane, LaneTile& lt) {
  uint16_t* tail = reinterpret_cast<uint16_t*>(st.tail) + h * (T * D);
  reinterpret_cast<uint2*>(tail + (long)pos * D)[lane] = reinterpret_cast<const uint2*>(xrow)[lane];       // 32 lanes x 8 B = one row
  if (pos + 1 != T) return -1;
  if ((long)tile * T + T > S_cap) return -1;          // cache full: never write past the head's capacity (callers check capacity at prefill)
  __syncwarp();
  stage_rows(ws, tail, D, T, lane);                   // rows written by this warp just now are visible to it after the barrier
  const int brow = (int)(h % n_base_rows);
  u32 b3w[8], b4w[8];
  load_base_words<KIND_V>(st.base3 + (long)brow * D, st.base4 + (long)brow * D, lane, b3w, b4w);
  return encode_tile_warp<KIND_V>(ws, T, b3w, b4w, lane, lt);
}
// Second half: the encoded tile goes to the head's streams, its escape bytes behind the bytes in use.
template <int KIND_V>
__device__ __forceinline__ void append_store(WarpScratch& ws, const gaac_store& st, const LaneTile& lt, long h, int tile, int total, long S_cap, long ovf_cap, int lane) {
  const long trow = h * S_cap + (long)tile * T;
  store_tile_payload<KIND_V>(lt, st.sm + trow * D, st.codes + trow * CB, lane);
  if (lane < T) st.flags[trow + lane] = (int)ws.fl[lane];
  const int used = st.ovf_used[h];
  store_tile_escapes<KIND_V>(ws, lt, st.ovf + h * ovf_cap + used, lane);
  __syncwarp();
  if (lane == 0) { st.tile_off[h * (S_cap / T) + tile] = used; st.ovf_used[h] = used + total; }
}

__global__ void __launch_bounds__(64) append_kv_kernel(const __grid_constant__ AppendParams p) {
  __shared__ __align__(16) WarpScratch scratch[2];
  __shared__ int s_fit[2];
  const int i = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sl = p.slot[i / p.n_kv];
  if (sl < 0) return;
  const long h = (long)sl * p.n_kv + i % p.n_kv;
  const int pos = p.tail_len[h], tile = p.seq_len[h] / T;
  LaneTile lt;
  const gaac_store& st = warp == 0 ? p.K : p.V;
  const int total = warp == 0 ? append_encode<0>(scratch[0], p.K, p.k_new + (long)i * D, h, pos, tile, p.S_cap, p.n_base_rows, lane, lt)
                              : append_encode<1>(scratch[1], p.V, p.v_new + (long)i * D, h, pos, tile, p.S_cap, p.n_base_rows, lane, lt);
  // A tile whose escape bytes (plus the 8 bytes a reader may touch behind them) do not fit what is left of the head's escape
  // stream is not stored, for K and V alike: nothing is written outside the head's share, the counters stay, *err counts it.
  if (lane == 0) s_fit[warp] = total < 0 || (long)st.ovf_used[h] + total + 8 <= p.ovf_cap;
  __syncthreads();                                    // both warps have read the counters
  const bool fits = s_fit[0] && s_fit[1];
  if (total >= 0 && fits) {
    if (warp == 0) append_store<0>(scratch[0], p.K, lt, h, tile, total, p.S_cap, p.ovf_cap, lane);
    else append_store<1>(scratch[1], p.V, lt, h, tile, total, p.S_cap, p.ovf_cap, lane);
  }
  if (threadIdx.x == 0) {
    const int t = pos + 1, full = (t == T);
    if (full && !fits) { if (p.err) atomicAdd(p.err, 1); return; }
    if (full && (long)tile * T + T > p.S_cap) return;   // cache full: the tile was not stored, keep the counters (the last tail row is overwritten next time)
    p.tail_len[h] = full ? 0 : t;
    if (full) p.seq_len[h] = p.seq_len[h] + T;
  }
}

// ------------------------------------------------------------------------------------------------ paged layout
struct PagedParams {
  gaac_paged st;
  const uint16_t *key, *value; long k_stride, v_stride;
  const int* ent; int* freeq;
};

__device__ __forceinline__ int pop_raw_tile(const gaac_paged& st, int lane) {
  int r = 0;
  if (lane == 0) {
    const int idx = atomicAdd(st.top, -1) - 1;
    if (idx >= 0) r = st.stack[idx]; else atomicAdd(st.err, 1);      // failed pop: tile 0 is written and the error counted
  }
  return __shfl_sync(FULL, r, 0);
}

// One warp per (entry, tile slot t = 2*kvh + kind).  grid = (E, 2*n_kv).
template <int KIND_V>
__device__ __forceinline__ void store_one(WarpScratch& ws, const PagedParams& p, int e, int t, int lane) {
  const gaac_paged& st = p.st;
  const int kvh = t >> 1, NT = 2 * st.n_kv;
  const int blk = p.ent[4 * e], tok0 = p.ent[4 * e + 1], off0 = p.ent[4 * e + 2], n = p.ent[4 * e + 3];
  if (blk < 0) { if (lane == 0) p.freeq[e * NT + t] = -1; return; }
  const long pt = (long)blk * NT + t;
  const int old = st.mt[pt];
  const bool have = old < 0, full = (off0 + n == T);
  const int r_old = have ? ~old : 0;
  const uint16_t* src = (KIND_V ? p.value : p.key) + (long)kvh * D;
  const long sstride = KIND_V ? p.v_stride : p.k_stride;
  uint16_t* rawp = reinterpret_cast<uint16_t*>(st.raw);
  int fits = 0, r = r_old;
  if (full) {
    // gather the tile: old rows from the raw tile (if any), new rows from this step's K/V
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const int c = lane + 32 * k, row = c >> 4, col = (c & 15) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row >= off0) v = *reinterpret_cast<const uint4*>(src + (long)(tok0 + row - off0) * sstride + col);
      else if (have) v = *reinterpret_cast<const uint4*>(rawp + ((long)r_old * T + row) * D + col);
      *reinterpret_cast<uint4*>(&ws.xs[row * XS_STRIDE + col]) = v;
    }
    u32 b3w[8], b4w[8];
    load_base_words<KIND_V>((KIND_V ? st.b3v : st.b3k) + kvh * D, (KIND_V ? st.b4v : st.b4k) + kvh * D, lane, b3w, b4w);
    LaneTile lt;
    const int total = encode_tile_warp<KIND_V>(ws, T, b3w, b4w, lane, lt);
    fits = total <= st.ovf_slot;
    if (fits) {
      uint8_t* base = st.buf + pt * st.TS;
      store_tile_payload<KIND_V>(lt, base, base + SLOT_CD_OFF, lane);
      if (lane < T) reinterpret_cast<u32*>(base + SLOT_FL_OFF)[lane] = ws.fl[lane];
      store_tile_escapes<KIND_V>(ws, lt, base + SLOT_OVF_OFF, lane);
    }
  }
  if (!fits) {
    if (!have) r = pop_raw_tile(st, lane);
    // new rows, natural channel order, into raw tile r
    for (int c = lane; c < n * 16; c += 32) {
      const int row = off0 + (c >> 4), col = (c & 15) * 8;
      *reinterpret_cast<uint4*>(rawp + ((long)r * T + row) * D + col) = *reinterpret_cast<const uint4*>(src + (long)(tok0 + row - off0) * sstride + col);
    }
  }
  if (lane == 0) {
    st.mt[pt] = fits ? (int)pt : ~r;
    p.freeq[e * NT + t] = (fits && have) ? r_old : -1;
  }
}

__global__ void __launch_bounds__(32) paged_store_kernel(const __grid_constant__ PagedParams p) {
  __shared__ __align__(16) WarpScratch ws;
  const int e = blockIdx.x, t = blockIdx.y, lane = threadIdx.x;
  if (t & 1) store_one<1>(ws, p, e, t, lane); else store_one<0>(ws, p, e, t, lane);
}

__global__ void __launch_bounds__(256) free_tiles_kernel(const int* __restrict__ freeq, int n_items, int* __restrict__ stack, int* __restrict__ top) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n_items) return;
  const int r = freeq[i];
  if (r >= 0) { const int idx = atomicAdd(top, 1); stack[idx] = r; }
}

__global__ void __launch_bounds__(32) release_blocks_kernel(const int* __restrict__ blocks, int NT, int* __restrict__ mt, int* __restrict__ stack, int* __restrict__ top) {
  const long blk = blocks[blockIdx.x];
  for (int t = threadIdx.x; t < NT; t += 32) {
    const long pt = blk * NT + t;
    const int m = mt[pt];
    if (m < 0) { const int idx = atomicAdd(top, 1); stack[idx] = ~m; mt[pt] = (int)pt; }
  }
}

struct PagedDecodeParams { gaac_paged st; const int* pairs; uint16_t *sk, *sv; long row_stride; };

template <int KIND_V>
__device__ __forceinline__ void decode_block_one(WarpScratch& ws, const PagedDecodeParams& p, int e, int t, int lane) {
  const gaac_paged& st = p.st;
  const int kvh = t >> 1, NT = 2 * st.n_kv;
  const int blk = p.pairs[3 * e], row0 = p.pairs[3 * e + 1], nvalid = p.pairs[3 * e + 2];
  const long pt = (long)blk * NT + t;
  const int m = st.mt[pt];
  uint16_t* dst = (KIND_V ? p.sv : p.sk) + (long)row0 * p.row_stride + (long)kvh * D;
  if (m < 0) {
    const uint16_t* rawp = reinterpret_cast<const uint16_t*>(st.raw) + (long)(~m) * T * D;
    for (int c = lane; c < nvalid * 16; c += 32) {
      const int row = c >> 4, col = (c & 15) * 8;
      *reinterpret_cast<uint4*>(dst + (long)row * p.row_stride + col) = *reinterpret_cast<const uint4*>(rawp + row * D + col);
    }
    return;
  }
  const uint8_t* base = st.buf + pt * st.TS;
  u32 b3w[8], dw[8];
  load_base_deltas<KIND_V>((KIND_V ? st.b3v : st.b3k) + kvh * D, (KIND_V ? st.b4v : st.b4k) + kvh * D, lane, b3w, dw);
  PtrEsc esc{base + SLOT_OVF_OFF};
  decode_tile_warp<KIND_V>(ws, base, base + SLOT_CD_OFF, reinterpret_cast<const u32*>(base + SLOT_FL_OFF), esc, b3w, dw, lane);
  unstage_rows(ws, dst, p.row_stride, nvalid, lane);
}

__global__ void __launch_bounds__(32) paged_decode_blocks_kernel(const __grid_constant__ PagedDecodeParams p) {
  __shared__ __align__(16) WarpScratch ws;
  const int e = blockIdx.x, t = blockIdx.y, lane = threadIdx.x;
  if (t & 1) decode_block_one<1>(ws, p, e, t, lane); else decode_block_one<0>(ws, p, e, t, lane);
}

static int check_paged(const gaac_paged* st) {
  if (!st || !st->buf || !st->raw || !st->mt || !st->stack || !st->top || !st->err || !st->b3k || !st->b4k || !st->b3v || !st->b4v) return GAAC_E_ARG;
  if (st->n_kv <= 0 || st->n_kv > 32767) return GAAC_E_ARG;
  if (st->TS % 16 || st->TS != SLOT_OVF_OFF + st->ovf_slot || st->ovf_slot < 0) return GAAC_E_UNSUPPORTED;
  if (!aligned16(st->buf) || !aligned16(st->raw)) return GAAC_E_ALIGN;
  return GAAC_OK;
}

}  // namespace gaac

using namespace gaac;

extern "C" int gaac_append_kv(const gaac_store* K, const gaac_store* V, const void* k_new, const void* v_new, const int32_t* slot, int B, int n_kv,
                              int32_t* tail_len, int32_t* seq_len, int64_t S_cap, int64_t ovf_cap, int n_base_rows, int32_t* err, void* stream) {
  if (!K || !V || !k_new || !v_new || !slot || !tail_len || !seq_len) return GAAC_E_ARG;
  if (B <= 0 || n_kv <= 0 || S_cap <= 0 || S_cap % T || ovf_cap <= 0 || n_base_rows <= 0) return GAAC_E_ARG;
  for (const gaac_store* s : {K, V}) {
    if (!s->sm || !s->codes || !s->flags || !s->tile_off || !s->ovf || !s->ovf_used || !s->tail || !s->base3 || !s->base4) return GAAC_E_ARG;
    if (!aligned16(s->sm) || !aligned16(s->codes) || !aligned16(s->tail)) return GAAC_E_ALIGN;
  }
  if ((reinterpret_cast<uintptr_t>(k_new) & 7) || (reinterpret_cast<uintptr_t>(v_new) & 7)) return GAAC_E_ALIGN;
  AppendParams p{*K, *V, (const uint16_t*)k_new, (const uint16_t*)v_new, slot, n_kv, tail_len, seq_len, S_cap, ovf_cap, n_base_rows, err};
  append_kv_kernel<<<(unsigned)(B * n_kv), 64, 0, (cudaStream_t)stream>>>(p);
  return launch_status();
}

extern "C" int gaac_paged_store(const gaac_paged* st, const void* key, const void* value, int64_t k_stride, int64_t v_stride,
                                const int32_t* ent, int E, int32_t* freeq, void* stream) {
  if (int e = check_paged(st)) return e;
  if (!key || !value || !ent || !freeq || E < 0 || k_stride < (int64_t)st->n_kv * D || v_stride < (int64_t)st->n_kv * D) return GAAC_E_ARG;
  if (!aligned16(key) || !aligned16(value) || k_stride % 8 || v_stride % 8) return GAAC_E_ALIGN;
  if (E == 0) return GAAC_OK;
  PagedParams p{*st, (const uint16_t*)key, (const uint16_t*)value, k_stride, v_stride, ent, freeq};
  cudaStream_t s = (cudaStream_t)stream;
  paged_store_kernel<<<dim3((unsigned)E, (unsigned)(2 * st->n_kv)), 32, 0, s>>>(p);
  const int n = E * 2 * st->n_kv;
  free_tiles_kernel<<<(n + 255) / 256, 256, 0, s>>>(freeq, n, st->stack, st->top);
  return launch_status();
}

extern "C" int gaac_paged_release(const gaac_paged* st, const int32_t* blocks, int F, void* stream) {
  if (int e = check_paged(st)) return e;
  if (!blocks || F < 0) return GAAC_E_ARG;
  if (F == 0) return GAAC_OK;
  release_blocks_kernel<<<(unsigned)F, 32, 0, (cudaStream_t)stream>>>(blocks, 2 * st->n_kv, st->mt, st->stack, st->top);
  return launch_status();
}

extern "C" int gaac_paged_decode_blocks(const gaac_paged* st, const int32_t* pairs, int P, void* sk, void* sv, int64_t row_stride, void* stream) {
  if (int e = check_paged(st)) return e;
  if (!pairs || !sk || !sv || P < 0 || row_stride < (int64_t)st->n_kv * D) return GAAC_E_ARG;
  if (!aligned16(sk) || !aligned16(sv) || row_stride % 8) return GAAC_E_ALIGN;
  if (P == 0) return GAAC_OK;
  PagedDecodeParams p{*st, pairs, (uint16_t*)sk, (uint16_t*)sv, row_stride};
  paged_decode_blocks_kernel<<<dim3((unsigned)P, (unsigned)(2 * st->n_kv)), 32, 0, (cudaStream_t)stream>>>(p);
  return launch_status();
}

extern "C" const char* gaac_status_string(int status) {
  switch (status) {
    case GAAC_OK: return "ok";
    case GAAC_E_ARG: return "invalid argument (null pointer, bad size or inconsistent sizes)";
    case GAAC_E_UNSUPPORTED: return "unsupported configuration (GQA group must be 1..8, head_dim 128, tile stride a multiple of 16)";
    case GAAC_E_ALIGN: return "a buffer is not aligned as required";
    case GAAC_E_LAUNCH: return "CUDA launch failed";
    case GAAC_E_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" int gaac_abi_version(void) { return 4; }
