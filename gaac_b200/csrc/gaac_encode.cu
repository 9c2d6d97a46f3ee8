// Block encoder, escape-stream compaction, page decoder and calibration kernels (sm_100a).
#include "gaac_api.cuh"
#include "gaac_warp.cuh"

namespace gaac {

constexpr int ENC_WARPS = 4;          // warps per CTA
constexpr int ENC_TILES_PER_WARP = 4; // consecutive work items of one warp share the head's base words

// One warp per (head, tile).  grid = (ceil(ntiles / (ENC_WARPS*ENC_TILES_PER_WARP)), H).  Token t of head h is read at
// x + h * x_head_stride + t * x_row_stride (bf16 elements): head-major [H, S_in, 128] or token-major [L, n_kv, 128] input.
template <int KIND_V>
__global__ void __launch_bounds__(ENC_WARPS * 32) encode_tiles_kernel(
    const uint16_t* __restrict__ x, long S, long x_head_stride, long x_row_stride, long S_pad, const uint8_t* __restrict__ base3,
    const uint8_t* __restrict__ base4, const int* __restrict__ bidx, int n_kv, uint8_t* __restrict__ sm, uint8_t* __restrict__ codes,
    int* __restrict__ flags, uint8_t* __restrict__ slots, int* __restrict__ tile_bytes, int ntiles) {
  __shared__ __align__(16) WarpScratch scratch[2][ENC_WARPS];       // two per warp: the next tile's rows arrive while this one is encoded
  __shared__ __align__(16) uint8_t esc_stage[ENC_WARPS][TILE_MAX_ESC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long h = blockIdx.y;
  const int brow = bidx ? bidx[h] : (int)(h % n_kv);
  u32 b3w[8], b4w[8];
  load_base_words<KIND_V>(base3 + (long)brow * D, base4 + (long)brow * D, lane, b3w, b4w);
  const int tile0 = blockIdx.x * (ENC_WARPS * ENC_TILES_PER_WARP) + warp;
  const uint16_t* xh = x + h * x_head_stride;
  auto fetch = [&](int i) {                           // rows of the warp's i-th tile into scratch[i & 1]
    const long row0 = (long)(tile0 + i * ENC_WARPS) * T;
    stage_rows_async(scratch[i & 1][warp], xh + row0 * x_row_stride, x_row_stride, (int)min((long)T, S - row0), lane);
    async_commit();
  };
  if (tile0 < ntiles) fetch(0);
  for (int i = 0; i < ENC_TILES_PER_WARP; i++) {
    const int tile = tile0 + i * ENC_WARPS;
    if (tile >= ntiles) break;                       // warp-uniform
    const bool more = i + 1 < ENC_TILES_PER_WARP && tile + ENC_WARPS < ntiles;
    __syncwarp();                                    // the other scratch was read by the tile before this one
    if (more) { fetch(i + 1); async_wait<1>(); } else async_wait<0>();
    WarpScratch& ws = scratch[i & 1][warp];
    const long row0 = (long)tile * T;
    const int nvalid = (int)min((long)T, S - row0);
    LaneTile lt;
    const int total = encode_tile_warp<KIND_V>(ws, nvalid, b3w, b4w, lane, lt);
    const long trow = h * S_pad + row0;
    store_tile_payload<KIND_V>(lt, sm + trow * D, codes + trow * CB, lane);
    if (lane < T) flags[trow + lane] = (int)ws.fl[lane];
    // escape bytes: gathered in shared memory with byte stores (every lane at its own positions), then written to the tile's
    // scratch slot as whole words by neighbouring lanes, so the slot costs one or two coalesced stores instead of ~50 byte stores
    store_tile_escapes<KIND_V>(ws, lt, esc_stage[warp], lane);
    __syncwarp();
    {
      u32* dst = reinterpret_cast<u32*>(slots + (h * ntiles + tile) * (long)TILE_MAX_ESC);
      const u32* src = reinterpret_cast<const u32*>(esc_stage[warp]);
      for (int k = lane; 4 * k < total; k += 32) dst[k] = src[k];
    }
    if (lane == 0) tile_bytes[h * ntiles + tile] = total;
  }
}

// Exclusive prefix of tile_bytes per head.  One CTA of 1024 threads per head, four tiles per thread and pass: a 64K-token
// head (4096 tiles) is one pass of two warp scans.
constexpr int SCAN_THREADS = 1024;
__global__ void __launch_bounds__(SCAN_THREADS) tile_scan_kernel(const int* __restrict__ tile_bytes, int ntiles, int* __restrict__ tile_off,
                                                                  long tile_off_stride, int* __restrict__ head_bytes) {
  __shared__ int wsum[32];
  __shared__ int carry_s, pass_total;
  const long h = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < ntiles; base += 4 * SCAN_THREADS) {
    const int i0 = base + 4 * tid;
    int v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) v[k] = i0 + k < ntiles ? tile_bytes[h * ntiles + i0 + k] : 0;
    const int s = v[0] + v[1] + v[2] + v[3];
    int inc = s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { int u = __shfl_up_sync(FULL, inc, d); if (lane >= d) inc += u; }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int w = wsum[lane];
      int winc = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) { int u = __shfl_up_sync(FULL, winc, d); if (lane >= d) winc += u; }
      wsum[lane] = winc - w;                         // exclusive prefix over the warps
      if (lane == 31) pass_total = winc;
    }
    __syncthreads();
    int off = carry_s + wsum[warp] + inc - s;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      if (i0 + k < ntiles) tile_off[h * tile_off_stride + i0 + k] = off;
      off += v[k];
    }
    __syncthreads();
    if (tid == 0) carry_s += pass_total;
    __syncthreads();
  }
  if (tid == 0 && head_bytes) head_bytes[h] = carry_s;
}

// head_start[0..H] = exclusive prefix of head_bytes (one small CTA; H is the number of cache heads).
__global__ void __launch_bounds__(256) head_prefix_kernel(const int* __restrict__ head_bytes, int H, int* __restrict__ head_start) {
  __shared__ int wsum[8];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { carry_s = 0; head_start[0] = 0; }
  __syncthreads();
  for (int base = 0; base < H; base += 256) {
    const int i = base + tid;
    const int v = i < H ? head_bytes[i] : 0;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { int u = __shfl_up_sync(FULL, inc, d); if (lane >= d) inc += u; }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; w++) woff += wsum[w];
    const int carry = carry_s;
    if (i < H) head_start[i + 1] = carry + woff + inc;
    __syncthreads();
    if (tid == 255) carry_s = carry + woff + inc;
    __syncthreads();
  }
}

// One warp per (head, tile): slot -> ovf[head_start[h] + tile_off[h, tile]]; optionally the per-row escape offsets
// ovf_off[h, row] = tile_off[h, tile] + (escape bytes of the tile's earlier rows), recomputed from the tag words.
__global__ void __launch_bounds__(128) compact_copy_kernel(const uint8_t* __restrict__ slots, const int* __restrict__ tile_bytes, int ntiles,
                                                            const int* __restrict__ tile_off, long tile_off_stride,
                                                            const int* __restrict__ head_start, long head_stride, uint8_t* __restrict__ ovf, long n_items,
                                                            const int* __restrict__ flags, long S, long S_pad, int* __restrict__ ovf_off, int zero_pad,
                                                            long ovf_cap, long head_cap, int* __restrict__ status) {
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int lane = threadIdx.x & 31;
  const long h = item / ntiles, t = item % ntiles;
  const int n = tile_bytes[item];
  const int toff = tile_off[h * tile_off_stride + t];
  const uint8_t* src = slots + item * (long)TILE_MAX_ESC;
  // bounds: the whole stream must fit ovf_cap bytes (ovf_cap > 0), a head's part head_cap bytes (head_cap > 0), read padding
  // included; a tile that does not fit is not written and bit 0 of *status is set
  const long at = (head_start ? (long)head_start[h] : h * head_stride) + toff;        // no table: head h's stream starts at h * head_stride
  const bool fits = (ovf_cap <= 0 || at + n + zero_pad <= ovf_cap) && (head_cap <= 0 || (long)toff + n + zero_pad <= head_cap);
  if (fits) { uint8_t* dst = ovf + at; for (int i = lane; i < n; i += 32) dst[i] = src[i]; }
  else if (lane == 0 && status) atomicOr(status, 1);
  if (zero_pad && head_cap <= 0 && head_start && item == 0 && lane < zero_pad) {                                    // over-read padding behind the last head (packed stream)
    const long end = (long)head_start[n_items / ntiles];
    if (ovf_cap <= 0 || end + zero_pad <= ovf_cap) ovf[end + lane] = 0;
    else if (lane == 0 && status) atomicOr(status, 1);
  }
  if (ovf_off) {
    const long row = t * T + (lane & 15);
    const int sz = (lane < T && row < S) ? row_esc_bytes((u32)flags[h * S_pad + row]) : 0;
    int inc = sz;
#pragma unroll
    for (int d = 1; d < T; d <<= 1) { int v = __shfl_up_sync(FULL, inc, d); if (lane >= d) inc += v; }
    if (lane < T && row < S) ovf_off[h * S + row] = toff + inc - sz;
  }
}

// One warp per (head, tile): compressed tile -> bf16 rows.
template <int KIND_V>
__global__ void __launch_bounds__(ENC_WARPS * 32) decode_page_kernel(
    const uint8_t* __restrict__ sm, const uint8_t* __restrict__ codes, const int* __restrict__ flags, const int* __restrict__ tile_off,
    long tile_off_stride, const uint8_t* __restrict__ ovf, const int* __restrict__ head_start, const uint8_t* __restrict__ base3,
    const uint8_t* __restrict__ base4, const int* __restrict__ bidx, int n_kv, long S, long S_pad, uint16_t* __restrict__ out, int ntiles) {
  __shared__ __align__(16) WarpScratch scratch[ENC_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long h = blockIdx.y;
  WarpScratch& ws = scratch[warp];
  const int brow = bidx ? bidx[h] : (int)(h % n_kv);
  u32 b3w[8], b4w[8];
  load_base_deltas<KIND_V>(base3 + (long)brow * D, base4 + (long)brow * D, lane, b3w, b4w);
  const int tile0 = blockIdx.x * (ENC_WARPS * ENC_TILES_PER_WARP);
  for (int i = 0; i < ENC_TILES_PER_WARP; i++) {
    const int tile = tile0 + i * ENC_WARPS + warp;
    if (tile >= ntiles) break;
    const long row0 = (long)tile * T, trow = h * S_pad + row0;
    PtrEsc esc{ovf + (long)head_start[h] + tile_off[h * tile_off_stride + tile]};
    __syncwarp();
    decode_tile_warp<KIND_V>(ws, sm + trow * D, codes + trow * CB, reinterpret_cast<const u32*>(flags + trow), esc, b3w, b4w, lane);
    unstage_rows(ws, out + (h * S + row0) * D, D, (int)min((long)T, S - row0), lane);
  }
}

// Exponent histogram: x [N, n_ch] bf16, hist [n_ch, 256] int64.  grid = (ceil(n_ch/128), row chunks); a thread owns one
// channel and keeps a private 256-bin histogram of 16-bit counters in shared memory, flushed with atomics.
constexpr int HIST_ROWS = 64;         // rows per CTA: short chunks put hundreds of CTAs on a 2048-token calibration sample (16-bit counters cannot overflow)
__global__ void __launch_bounds__(128) exponent_hist_kernel(const uint16_t* __restrict__ x, long N, long n_ch, unsigned long long* __restrict__ hist) {
  extern __shared__ unsigned short bins[];           // [256][128]: bin-major so a warp's increments spread over banks
  const int tid = threadIdx.x;
  const long c = (long)blockIdx.x * 128 + tid;
  for (int b = 0; b < 256; b++) bins[b * 128 + tid] = 0;
  const long r0 = (long)blockIdx.y * HIST_ROWS, r1 = min(N, r0 + HIST_ROWS);
  if (c < n_ch) {
    long r = r0;
    for (; r + 4 <= r1; r += 4) {                       // four independent loads in flight per thread
      const unsigned a0 = x[r * n_ch + c], a1 = x[(r + 1) * n_ch + c], a2 = x[(r + 2) * n_ch + c], a3 = x[(r + 3) * n_ch + c];
      bins[((a0 >> 7) & 0xFF) * 128 + tid]++; bins[((a1 >> 7) & 0xFF) * 128 + tid]++;
      bins[((a2 >> 7) & 0xFF) * 128 + tid]++; bins[((a3 >> 7) & 0xFF) * 128 + tid]++;
    }
    for (; r < r1; r++) bins[((x[r * n_ch + c] >> 7) & 0xFF) * 128 + tid]++;
  }
  if (c < n_ch)
    for (int b = 0; b < 256; b++) {
      unsigned v = bins[b * 128 + tid];
      if (v) atomicAdd(&hist[c * 256 + b], (unsigned long long)v);
    }
}

// One warp per histogram row: densest 8- and 16-wide window, first maximum wins.
__global__ void __launch_bounds__(128) bases_from_hist_kernel(const long long* __restrict__ hist, long n_rows, uint8_t* __restrict__ base3, uint8_t* __restrict__ base4) {
  __shared__ long long cs[4][257];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * 4 + warp;
  if (row >= n_rows) return;
  long long carry = 0;
  if (lane == 0) cs[warp][0] = 0;
  for (int b = 0; b < 256; b += 32) {
    long long v = hist[row * 256 + b + lane], inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { long long u = __shfl_up_sync(FULL, inc, d); if (lane >= d) inc += u; }
    cs[warp][b + lane + 1] = carry + inc;
    carry += __shfl_sync(FULL, inc, 31);
  }
  __syncwarp();
  for (int k = 0; k < 2; k++) {
    const int w = k ? 16 : 8;
    long long best = -1; int besti = 0;
    for (int s = lane; s <= 256 - w; s += 32) {
      long long v = cs[warp][s + w] - cs[warp][s];
      if (v > best) { best = v; besti = s; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      long long ob = __shfl_xor_sync(FULL, best, d); int oi = __shfl_xor_sync(FULL, besti, d);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0) (k ? base4 : base3)[row] = (uint8_t)besti;
  }
}

// Last step of a slot's prefill (one CTA): the prompt's remainder (L mod 16 rows) goes into the raw tails of the slot's heads,
// the heads' token counters are set, and the largest escape stream of the slot per kind is reported for the host's capacity
// check.  k_tok / v_tok: token-major rows, head h of token t at t * row_stride + h * 128 (bf16 elements).
__global__ void __launch_bounds__(256) prefill_finish_kernel(const uint16_t* __restrict__ k_tok, const uint16_t* __restrict__ v_tok, long row_stride, long L,
                                                              int n_kv, long h0, uint16_t* __restrict__ ktail, uint16_t* __restrict__ vtail,
                                                              int* __restrict__ seq_len, int* __restrict__ tail_len, int* __restrict__ used_k,
                                                              int* __restrict__ used_v, int* __restrict__ status) {
  const long n_full = L / T * T;
  const int rem = (int)(L - n_full), tid = threadIdx.x;
  const int per_kind = rem * n_kv * 16;                              // 16-byte pieces
  for (int i = tid; i < 2 * per_kind; i += blockDim.x) {
    const int kind = i >= per_kind, j = i - kind * per_kind;
    const int r = j / (n_kv * 16), h = (j >> 4) % n_kv, c = j & 15;
    const uint16_t* src = (kind ? v_tok : k_tok) + (n_full + r) * row_stride + h * D + c * 8;
    uint16_t* dst = (kind ? vtail : ktail) + ((h0 + h) * T + r) * D + c * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
  if (tid < n_kv) {
    seq_len[h0 + tid] = (int)n_full; tail_len[h0 + tid] = rem;
    if (n_full == 0) { used_k[h0 + tid] = 0; used_v[h0 + tid] = 0; }
  }
  __syncthreads();
  if (tid == 0) {
    int mk = 0, mv = 0;
    for (int h = 0; h < n_kv; h++) { mk = max(mk, used_k[h0 + h]); mv = max(mv, used_v[h0 + h]); }
    status[1] = mk; status[3] = mv;
  }
}

}  // namespace gaac

using namespace gaac;

extern "C" int gaac_encode_tiles(const void* x_bf16, int64_t H, int64_t S, int64_t S_in, int64_t S_pad,
                                 const uint8_t* base3, const uint8_t* base4, const int32_t* bidx, int n_kv, int kind,
                                 uint8_t* sm, uint8_t* codes, int32_t* flags, uint8_t* slots, int32_t* tile_bytes, void* stream) {
  if (!x_bf16 || !base3 || !base4 || !sm || !codes || !flags || !slots || !tile_bytes) return GAAC_E_ARG;
  if (H <= 0 || S <= 0 || S_in < S || S_pad < (S + T - 1) / T * T || S_pad % T || n_kv <= 0 || H > 65535 || (kind != GAAC_KIND_K && kind != GAAC_KIND_V)) return GAAC_E_ARG;
  if (!aligned16(x_bf16) || !aligned16(sm) || !aligned16(codes)) return GAAC_E_ALIGN;
  const int ntiles = (int)((S + T - 1) / T);
  dim3 grid((ntiles + ENC_WARPS * ENC_TILES_PER_WARP - 1) / (ENC_WARPS * ENC_TILES_PER_WARP), (unsigned)H);
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == GAAC_KIND_K)
    encode_tiles_kernel<0><<<grid, ENC_WARPS * 32, 0, st>>>((const uint16_t*)x_bf16, S, S_in * D, D, S_pad, base3, base4, bidx, n_kv, sm, codes, flags, slots, tile_bytes, ntiles);
  else
    encode_tiles_kernel<1><<<grid, ENC_WARPS * 32, 0, st>>>((const uint16_t*)x_bf16, S, S_in * D, D, S_pad, base3, base4, bidx, n_kv, sm, codes, flags, slots, tile_bytes, ntiles);
  return launch_status();
}

extern "C" int gaac_compact(const uint8_t* slots, const int32_t* tile_bytes, int64_t H, int64_t ntiles, const int32_t* head_start,
                            uint8_t* ovf, int32_t* tile_off, int64_t tile_off_stride, int32_t* head_bytes,
                            const int32_t* flags, int64_t S, int64_t S_pad, int32_t* ovf_off, void* stream) {
  if (!tile_bytes || !tile_off || H <= 0 || ntiles <= 0 || tile_off_stride < ntiles) return GAAC_E_ARG;
  if (head_start && (!ovf || !slots)) return GAAC_E_ARG;
  if (ovf_off && (!head_start || !flags || S <= 0 || S_pad < S)) return GAAC_E_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  tile_scan_kernel<<<(unsigned)H, SCAN_THREADS, 0, st>>>(tile_bytes, (int)ntiles, tile_off, tile_off_stride, head_bytes);
  if (head_start) {
    const long n_items = H * ntiles;
    compact_copy_kernel<<<(unsigned)((n_items + 3) / 4), 128, 0, st>>>(slots, tile_bytes, (int)ntiles, tile_off, tile_off_stride, head_start, 0, ovf, n_items,
                                                                    flags, S, S_pad, ovf_off, 0, 0, 0, nullptr);
  }
  return launch_status();
}

extern "C" int gaac_encode_begin(const void* x_bf16, int64_t H, int64_t S, int64_t S_in, int64_t S_pad,
                                 const uint8_t* base3, const uint8_t* base4, const int32_t* bidx, int n_kv, int kind,
                                 uint8_t* sm, uint8_t* codes, int32_t* flags, uint8_t* slots, int32_t* tile_bytes,
                                 int32_t* tile_off, int32_t* head_bytes, int32_t* head_start, void* stream) {
  if (!tile_off || !head_bytes || !head_start) return GAAC_E_ARG;
  if (int e = gaac_encode_tiles(x_bf16, H, S, S_in, S_pad, base3, base4, bidx, n_kv, kind, sm, codes, flags, slots, tile_bytes, stream)) return e;
  const int64_t ntiles = (S + T - 1) / T;
  if (int e = gaac_compact(nullptr, tile_bytes, H, ntiles, nullptr, nullptr, tile_off, ntiles, head_bytes, nullptr, 0, 0, nullptr, stream)) return e;
  return gaac_head_prefix(head_bytes, H, head_start, stream);
}

extern "C" int gaac_compact_copy(const uint8_t* slots, const int32_t* tile_bytes, int64_t H, int64_t ntiles, const int32_t* head_start, uint8_t* ovf,
                                 const int32_t* tile_off, int64_t tile_off_stride, const int32_t* flags, int64_t S, int64_t S_pad, int32_t* ovf_off,
                                 int zero_pad, int64_t ovf_cap, int64_t head_cap, int32_t* status, void* stream) {
  if (!slots || !tile_bytes || !head_start || !ovf || !tile_off || H <= 0 || ntiles <= 0 || tile_off_stride < ntiles || zero_pad < 0 || zero_pad > 32) return GAAC_E_ARG;
  if (ovf_cap < 0 || head_cap < 0) return GAAC_E_ARG;
  if (ovf_off && (!flags || S <= 0 || S_pad < S)) return GAAC_E_ARG;
  const long n_items = H * ntiles;
  compact_copy_kernel<<<(unsigned)((n_items + 3) / 4), 128, 0, (cudaStream_t)stream>>>(slots, tile_bytes, (int)ntiles, tile_off, tile_off_stride, head_start, 0, ovf,
                                                                                       n_items, flags, S, S_pad, ovf_off, zero_pad, ovf_cap, head_cap, status);
  return launch_status();
}

extern "C" int gaac_head_prefix(const int32_t* head_bytes, int64_t H, int32_t* head_start, void* stream) {
  if (!head_bytes || !head_start || H <= 0) return GAAC_E_ARG;
  head_prefix_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(head_bytes, (int)H, head_start);
  return launch_status();
}

extern "C" int gaac_decode_page(const uint8_t* sm, const uint8_t* codes, const int32_t* flags, const int32_t* tile_off, int64_t tile_off_stride,
                                const uint8_t* ovf, const int32_t* head_start, const uint8_t* base3, const uint8_t* base4, const int32_t* bidx,
                                int n_kv, int kind, int64_t H, int64_t S, int64_t S_pad, void* out_bf16, void* stream) {
  if (!sm || !codes || !flags || !tile_off || !ovf || !head_start || !base3 || !base4 || !out_bf16) return GAAC_E_ARG;
  if (H <= 0 || S <= 0 || S_pad < (S + T - 1) / T * T || S_pad % T || n_kv <= 0 || H > 65535 || (kind != GAAC_KIND_K && kind != GAAC_KIND_V)) return GAAC_E_ARG;
  if (!aligned16(sm) || !aligned16(codes) || !aligned16(out_bf16)) return GAAC_E_ALIGN;
  const int ntiles = (int)((S + T - 1) / T);
  dim3 grid((ntiles + ENC_WARPS * ENC_TILES_PER_WARP - 1) / (ENC_WARPS * ENC_TILES_PER_WARP), (unsigned)H);
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == GAAC_KIND_K)
    decode_page_kernel<0><<<grid, ENC_WARPS * 32, 0, st>>>(sm, codes, flags, tile_off, tile_off_stride, ovf, head_start, base3, base4, bidx, n_kv, S, S_pad, (uint16_t*)out_bf16, ntiles);
  else
    decode_page_kernel<1><<<grid, ENC_WARPS * 32, 0, st>>>(sm, codes, flags, tile_off, tile_off_stride, ovf, head_start, base3, base4, bidx, n_kv, S, S_pad, (uint16_t*)out_bf16, ntiles);
  return launch_status();
}

extern "C" int gaac_exponent_hist(const void* x_bf16, int64_t N, int64_t n_ch, long long* hist, void* stream) {
  if (!x_bf16 || !hist || N <= 0 || n_ch <= 0) return GAAC_E_ARG;
  cudaFuncSetAttribute(exponent_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * 128 * 2);   // per device; cheap
  dim3 grid((unsigned)((n_ch + 127) / 128), (unsigned)((N + HIST_ROWS - 1) / HIST_ROWS));
  exponent_hist_kernel<<<grid, 128, 256 * 128 * 2, (cudaStream_t)stream>>>((const uint16_t*)x_bf16, N, n_ch, (unsigned long long*)hist);
  return launch_status();
}

extern "C" int gaac_bases_from_hist(const long long* hist, int64_t n_rows, uint8_t* base3, uint8_t* base4, void* stream) {
  if (!hist || !base3 || !base4 || n_rows <= 0) return GAAC_E_ARG;
  bases_from_hist_kernel<<<(unsigned)((n_rows + 3) / 4), 128, 0, (cudaStream_t)stream>>>(hist, n_rows, base3, base4);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------- slot cache: whole-prompt prefill
constexpr int CACHE_READ_PAD = 8;      // bytes kept free behind a head's escape bytes (the readers may touch them)

extern "C" size_t gaac_cache_prefill_scratch_bytes(int64_t L, int n_kv) {
  const size_t items = (size_t)(L > 0 ? L / T : 0) * (size_t)(n_kv > 0 ? n_kv : 0);
  return 2 * items * (TILE_MAX_ESC + sizeof(int32_t)) + 256;
}

extern "C" int gaac_cache_prefill(const gaac_store* K, const gaac_store* V, const void* k_tok, const void* v_tok, int64_t L, int64_t row_stride, int slot,
                                  int n_kv, int32_t* tail_len, int32_t* seq_len, int64_t S_cap, int64_t ovf_cap, int n_base_rows, uint8_t* scratch,
                                  size_t scratch_bytes, int32_t* status, int copy_only, void* stream) {
  if (!K || !V || !tail_len || !seq_len || !scratch || !status || (!copy_only && L > 0 && (!k_tok || !v_tok))) return GAAC_E_ARG;
  if (L < 0 || L > S_cap || S_cap % T || row_stride < (int64_t)n_kv * D || slot < 0 || n_kv <= 0 || n_kv > 256 || ovf_cap <= CACHE_READ_PAD ||
      n_base_rows <= 0 || n_base_rows % n_kv)
    return GAAC_E_ARG;
  for (const gaac_store* s : {K, V}) {
    if (!s->sm || !s->codes || !s->flags || !s->tile_off || !s->ovf || !s->ovf_used || !s->tail || !s->base3 || !s->base4) return GAAC_E_ARG;
    if (!aligned16(s->sm) || !aligned16(s->codes) || !aligned16(s->tail)) return GAAC_E_ALIGN;
  }
  if (!copy_only && (!aligned16(k_tok) || !aligned16(v_tok) || (row_stride * 2) % 16)) return GAAC_E_ALIGN;
  if (scratch_bytes < gaac_cache_prefill_scratch_bytes(L, n_kv)) return GAAC_E_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const long h0 = (long)slot * n_kv;
  const int ntiles = (int)(L / T);
  const long S = (long)ntiles * T, tiles_cap = S_cap / T, n_items = (long)n_kv * ntiles;
  // scratch: escape slots of K, of V, then the tile sizes of K, of V
  uint8_t* slots[2] = {scratch, scratch + n_items * TILE_MAX_ESC};
  int32_t* tbytes[2] = {reinterpret_cast<int32_t*>(scratch + 2 * n_items * TILE_MAX_ESC), reinterpret_cast<int32_t*>(scratch + 2 * n_items * TILE_MAX_ESC) + n_items};
  if (copy_only) { cudaMemsetAsync(status, 0, 4, st); cudaMemsetAsync(status + 2, 0, 4, st); }
  else cudaMemsetAsync(status, 0, 16, st);
  const gaac_store* side[2] = {K, V};
  const void* tok[2] = {k_tok, v_tok};
  for (int kind = 0; kind < 2 && ntiles > 0; kind++) {
    const gaac_store* s = side[kind];
    int32_t* toff = s->tile_off + h0 * tiles_cap;
    if (!copy_only) {
      const uint8_t* b3 = s->base3 + (h0 % n_base_rows) * D; const uint8_t* b4 = s->base4 + (h0 % n_base_rows) * D;      // consecutive heads, consecutive rows
      dim3 grid((ntiles + ENC_WARPS * ENC_TILES_PER_WARP - 1) / (ENC_WARPS * ENC_TILES_PER_WARP), (unsigned)n_kv);
      if (kind == 0)
        encode_tiles_kernel<0><<<grid, ENC_WARPS * 32, 0, st>>>((const uint16_t*)tok[kind], S, D, row_stride, S_cap, b3, b4, nullptr, n_kv, s->sm + h0 * S_cap * D,
                                                               s->codes + h0 * S_cap * CB, s->flags + h0 * S_cap, slots[kind], tbytes[kind], ntiles);
      else
        encode_tiles_kernel<1><<<grid, ENC_WARPS * 32, 0, st>>>((const uint16_t*)tok[kind], S, D, row_stride, S_cap, b3, b4, nullptr, n_kv, s->sm + h0 * S_cap * D,
                                                               s->codes + h0 * S_cap * CB, s->flags + h0 * S_cap, slots[kind], tbytes[kind], ntiles);
      tile_scan_kernel<<<(unsigned)n_kv, SCAN_THREADS, 0, st>>>(tbytes[kind], ntiles, toff, tiles_cap, s->ovf_used + h0);
    }
    compact_copy_kernel<<<(unsigned)((n_items + 3) / 4), 128, 0, st>>>(slots[kind], tbytes[kind], ntiles, toff, tiles_cap, nullptr, ovf_cap, s->ovf + h0 * ovf_cap, n_items,
                                                                    nullptr, 0, 0, nullptr, 0, 0, ovf_cap - CACHE_READ_PAD, status + 2 * kind);
  }
  if (!copy_only)
    prefill_finish_kernel<<<1, 256, 0, st>>>((const uint16_t*)k_tok, (const uint16_t*)v_tok, row_stride, L, n_kv, h0, (uint16_t*)K->tail, (uint16_t*)V->tail,
                                             seq_len, tail_len, K->ovf_used, V->ovf_used, status);
  return launch_status();
}
