// Warp-level tile encode / decode built on the lane-level functions of gaac_tile.h.
// One warp owns one 16-token tile.  Shared by the page encoder, the slot-cache append and the paged store kernels.
#pragma once
#include <cuda_runtime.h>
#include "gaac_tile.h"

namespace gaac {

constexpr int XS_STRIDE = 136;                      // u16 per staged row: 272 B keeps 16-byte alignment and spreads banks
constexpr unsigned FULL = 0xffffffffu;

// Per-warp scratch in shared memory.
struct WarpScratch {
  uint16_t xs[T * XS_STRIDE];                        // staged tile, natural channel order
  uint8_t tag[T][16];                                // tier tag per (row, group)
  u32 fl[T];                                         // tag word per row
  int rowoff[T];                                     // escape offset of each row inside the tile
};

// Escape byte reader over plain memory (global or shared).
struct PtrEsc {
  const uint8_t* p;
  __host__ __device__ u32 byte(int pos) const { return p[pos]; }
  __host__ __device__ u64 bytes5(int pos) const {
    return (u64)p[pos] | ((u64)p[pos + 1] << 8) | ((u64)p[pos + 2] << 16) | ((u64)p[pos + 3] << 24) | ((u64)p[pos + 4] << 32);
  }
};

// Encoded tile held in registers, one lane's share.  8 groups per lane for both kinds:
//   K: idx = 4*o + g  -> row 8o + (lane>>2), group 4*(lane&3) + g          V: idx = 2*t + g -> row tok(t), group 2*(lane>>2) + g
struct LaneTile {
  u32 sm[16];        // K: [o][8] words;  V: [t][4] words
  u32 cd[6];         // K: [o][3] words;  V: 192 code bits (4 token slots x 48)
  u64 esc[8];
  u32 tags;          // 2 bits per idx
};

__device__ __forceinline__ int v_tok(int j, int t) { return 2 * j + (t & 1) + 8 * (t >> 1); }
__device__ __forceinline__ int lane_row(int kind_v, int lane, int idx) { return kind_v ? v_tok(lane & 3, idx >> 1) : 8 * (idx >> 2) + (lane >> 2); }
__device__ __forceinline__ int lane_group(int kind_v, int lane, int idx) { return kind_v ? 2 * (lane >> 2) + (idx & 1) : 4 * (lane & 3) + (idx & 3); }

// Stage rows [row0, row0+16) of a [*, 128] bf16 matrix into ws.xs; rows >= nvalid are zero-filled.
__device__ __forceinline__ void stage_rows(WarpScratch& ws, const uint16_t* src, long row_stride, int nvalid, int lane) {
#pragma unroll
  for (int k = 0; k < 8; k++) {
    int c = lane + 32 * k, row = c >> 4, col = (c & 15) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < nvalid) v = *reinterpret_cast<const uint4*>(src + (long)row * row_stride + col);
    *reinterpret_cast<uint4*>(&ws.xs[row * XS_STRIDE + col]) = v;
  }
}

// The same staging with asynchronous 16-byte copies (rows >= nvalid are zero-filled by the copy unit): the caller commits the
// group and waits for it before encode_tile_warp, so the rows of the next tile travel while the current one is encoded.
__device__ __forceinline__ void stage_rows_async(WarpScratch& ws, const uint16_t* src, long row_stride, int nvalid, int lane) {
  // piece k of a lane: row 2k + (lane >> 4), columns 8 * (lane & 15) .. +7: one source and one destination address per lane, a
  // fixed step per piece
  const int r0 = lane >> 4, col = (lane & 15) * 8;
  const uint16_t* g = src + (long)r0 * row_stride + col;
  const unsigned d = (unsigned)__cvta_generic_to_shared(&ws.xs[r0 * XS_STRIDE + col]);
  const long step = 2 * row_stride;
  if (nvalid == T) {
#pragma unroll
    for (int k = 0; k < 8; k++)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d + k * (2 * XS_STRIDE * 2)), "l"(g + k * step) : "memory");
  } else {
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const bool live = 2 * k + r0 < nvalid;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d + k * (2 * XS_STRIDE * 2)), "l"(live ? g + k * step : src), "r"(live ? 16 : 0) : "memory");
    }
  }
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Encode the staged tile.  Rows >= nvalid become empty rows (sm = 0, codes = 0, tag word 0).  On return every lane holds
// its share in `lt`, ws.fl / ws.rowoff are filled and the tile's escape byte count is returned (same in all lanes).
template <int KIND_V>
__device__ __forceinline__ int encode_tile_warp(WarpScratch& ws, int nvalid, const u32* b3w, const u32* b4w, int lane, LaneTile& lt) {
  const int j = lane & 3, r = lane >> 2;
  lt.tags = 0;
  __syncwarp();                                      // staged rows visible; previous tile's scratch no longer in use
  if (!KIND_V) {
#pragma unroll
    for (int o = 0; o < 2; o++) {
      int row = 8 * o + r; u32 t8 = 0;
      if (row < nvalid) encode_k_lane(&ws.xs[row * XS_STRIDE], j, b3w, b4w, &lt.sm[8 * o], &lt.cd[3 * o], t8, &lt.esc[4 * o]);
      else {
#pragma unroll
        for (int i = 0; i < 8; i++) lt.sm[8 * o + i] = 0;
        lt.cd[3 * o] = lt.cd[3 * o + 1] = lt.cd[3 * o + 2] = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) lt.esc[4 * o + i] = 0;
      }
      lt.tags |= t8 << (8 * o);
    }
  } else {
    u64 c48[4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
      int row = v_tok(j, t); u32 t4 = 0; c48[t] = 0;
      if (row < nvalid) encode_v_lane(&ws.xs[row * XS_STRIDE], r, b3w, b4w, &lt.sm[4 * t], c48[t], t4, &lt.esc[2 * t]);
      else {
#pragma unroll
        for (int i = 0; i < 4; i++) lt.sm[4 * t + i] = 0;
        lt.esc[2 * t] = lt.esc[2 * t + 1] = 0;
      }
      lt.tags |= t4 << (4 * t);
    }
    lt.cd[0] = (u32)c48[0];
    lt.cd[1] = (u32)(c48[0] >> 32) | ((u32)c48[1] << 16);
    lt.cd[2] = (u32)(c48[1] >> 16);
    lt.cd[3] = (u32)c48[2];
    lt.cd[4] = (u32)(c48[2] >> 32) | ((u32)c48[3] << 16);
    lt.cd[5] = (u32)(c48[3] >> 16);
  }
  __syncwarp();                                      // xs fully read before the scratch tables are reused by a later tile
#pragma unroll
  for (int idx = 0; idx < 8; idx++) ws.tag[lane_row(KIND_V, lane, idx)][lane_group(KIND_V, lane, idx)] = (uint8_t)((lt.tags >> (2 * idx)) & 3u);
  __syncwarp();
  int total;
  {
    u32 fl = 0; int sz = 0;
    if (lane < T) {
      const u32* tw = reinterpret_cast<const u32*>(ws.tag[lane]);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        u32 w = tw[q];                               // four tags, one per byte
        fl |= ((w & 3u) | ((w >> 6) & 0xCu) | ((w >> 12) & 0x30u) | ((w >> 18) & 0xC0u)) << (8 * q);
      }
      sz = row_esc_bytes(fl);
    }
    int inc = sz;
#pragma unroll
    for (int d = 1; d < T; d <<= 1) { int v = __shfl_up_sync(FULL, inc, d); if (lane >= d) inc += v; }
    if (lane < T) { ws.fl[lane] = fl; ws.rowoff[lane] = inc - sz; }
    total = __shfl_sync(FULL, inc, T - 1);
  }
  __syncwarp();
  return total;
}

// Write one lane's sign/mantissa and code bytes of the tile (tile-relative destinations).
template <int KIND_V>
__device__ __forceinline__ void store_tile_payload(const LaneTile& lt, uint8_t* sm_dst, uint8_t* cd_dst, int lane) {
  if (!KIND_V) {
#pragma unroll
    for (int o = 0; o < 2; o++) {
      uint4* s = reinterpret_cast<uint4*>(sm_dst + o * 1024 + 32 * lane);
      s[0] = make_uint4(lt.sm[8 * o], lt.sm[8 * o + 1], lt.sm[8 * o + 2], lt.sm[8 * o + 3]);
      s[1] = make_uint4(lt.sm[8 * o + 4], lt.sm[8 * o + 5], lt.sm[8 * o + 6], lt.sm[8 * o + 7]);
      u32* c = reinterpret_cast<u32*>(cd_dst + o * 384 + 12 * lane);
      c[0] = lt.cd[3 * o]; c[1] = lt.cd[3 * o + 1]; c[2] = lt.cd[3 * o + 2];
    }
  } else {
#pragma unroll
    for (int t = 0; t < 4; t++)
      *reinterpret_cast<uint4*>(sm_dst + 64 * lane + 16 * t) = make_uint4(lt.sm[4 * t], lt.sm[4 * t + 1], lt.sm[4 * t + 2], lt.sm[4 * t + 3]);
    uint2* c = reinterpret_cast<uint2*>(cd_dst + 24 * lane);
    c[0] = make_uint2(lt.cd[0], lt.cd[1]); c[1] = make_uint2(lt.cd[2], lt.cd[3]); c[2] = make_uint2(lt.cd[4], lt.cd[5]);
  }
}

// Write the tile's escape bytes at esc_dst + (tile-relative position), rows in token order, groups ascending.
template <int KIND_V>
__device__ __forceinline__ void store_tile_escapes(const WarpScratch& ws, const LaneTile& lt, uint8_t* esc_dst, int lane) {
  if (lt.tags == 0) return;
  // A lane's groups come in runs of consecutive groups of one row (K: 2 rows x 4 groups, V: 4 rows x 2 groups): the position of a
  // run's first escape byte is computed once, the groups of the run then follow one another in the row's escape bytes.
  constexpr int RUN = KIND_V ? 2 : 4;
#pragma unroll
  for (int base = 0; base < 8; base += RUN) {
    const u32 tr = (lt.tags >> (2 * base)) & ((1u << (2 * RUN)) - 1u);
    if (tr) {
      const int row = lane_row(KIND_V, lane, base), g0 = lane_group(KIND_V, lane, base);
      uint8_t* d = esc_dst + ws.rowoff[row] + esc_prefix(ws.fl[row], 2 * g0);
#pragma unroll
      for (int i = 0; i < RUN; i++) {
        const u32 tag = (tr >> (2 * i)) & 3u;
        if (tag) {
          const u64 e = lt.esc[base + i];
          d[0] = (uint8_t)e;
          if (tag & 2u) { d[1] = (uint8_t)(e >> 8); d[2] = (uint8_t)(e >> 16); d[3] = (uint8_t)(e >> 24); d[4] = (uint8_t)(e >> 32); }
          d += tag_esc_bytes(tag);
        }
      }
    }
  }
}

// Load the lane's base words for a (kind, base row).
template <int KIND_V>
__device__ __forceinline__ void load_base_words(const uint8_t* b3row, const uint8_t* b4row, int lane, u32* b3w, u32* b4w) {
  if (!KIND_V) { k_base_words(b3row, lane & 3, b3w); k_base_words(b4row, lane & 3, b4w); }
  else { v_base_words(b3row, lane >> 2, b3w); v_base_words(b4row, lane >> 2, b4w); }
}
// Same, but the second table is returned as the difference (4-bit base word - 3-bit base word) that decode_group wants.
template <int KIND_V>
__device__ __forceinline__ void load_base_deltas(const uint8_t* b3row, const uint8_t* b4row, int lane, u32* b3w, u32* dw) {
  load_base_words<KIND_V>(b3row, b4row, lane, b3w, dw);
#pragma unroll
  for (int i = 0; i < (KIND_V ? 4 : 8); i++) dw[i] -= b3w[i];
}

// Rebuild a compressed tile into ws.xs (natural channel order, bf16 bits).  sm/cd/fl: tile-relative sources;
// esc: reader positioned at the tile's first escape byte.
template <int KIND_V, class Esc>
__device__ __forceinline__ void decode_tile_warp(WarpScratch& ws, const uint8_t* sm_src, const uint8_t* cd_src, const u32* fl_src,
                                                 const Esc& esc, const u32* b3w, const u32* dw, int lane) {
  const int j = lane & 3, r = lane >> 2;
  {
    u32 fl = lane < T ? fl_src[lane] : 0u; int sz = row_esc_bytes(fl), inc = sz;
#pragma unroll
    for (int d = 1; d < T; d <<= 1) { int v = __shfl_up_sync(FULL, inc, d); if (lane >= d) inc += v; }
    if (lane < T) { ws.fl[lane] = fl; ws.rowoff[lane] = inc - sz; }
  }
  __syncwarp();
  if (!KIND_V) {
#pragma unroll
    for (int o = 0; o < 2; o++) {
      const int row = 8 * o + r;
      const uint4* s = reinterpret_cast<const uint4*>(sm_src + o * 1024 + 32 * lane);
      uint4 s0 = s[0], s1 = s[1];
      const u32 sm[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const u32* c = reinterpret_cast<const u32*>(cd_src + o * 384 + 12 * lane);
      const u32 cd[3] = {c[0], c[1], c[2]};
      const u32 fl = ws.fl[row];
      int pos = ws.rowoff[row] + esc_prefix(fl, 8 * j);
#pragma unroll
      for (int g = 0; g < 4; g++) {
        u32 out[4];
        decode_group(sm[2 * g], sm[2 * g + 1], k_group_codes(cd, g), (fl >> (8 * j + 2 * g)) & 3u, pos, esc,
                     b3w[2 * g], b3w[2 * g + 1], dw[2 * g], dw[2 * g + 1], out);
#pragma unroll
        for (int h = 0; h < 2; h++) {
          int s_ = 2 * g + h;
          u32* x = reinterpret_cast<u32*>(&ws.xs[row * XS_STRIDE + 16 * s_ + 2 * j]);
          x[0] = out[2 * h]; x[4] = out[2 * h + 1];
        }
      }
    }
  } else {
    const uint2* c2 = reinterpret_cast<const uint2*>(cd_src + 24 * lane);
    uint2 ca = c2[0], cb = c2[1], cc = c2[2];
    const u32 cd[6] = {ca.x, ca.y, cb.x, cb.y, cc.x, cc.y};
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int row = v_tok(j, t);
      uint4 s = *reinterpret_cast<const uint4*>(sm_src + 64 * lane + 16 * t);
      const u32 sm[4] = {s.x, s.y, s.z, s.w};
      const u32 fl = ws.fl[row];
      int pos = ws.rowoff[row] + esc_prefix(fl, 4 * r);
#pragma unroll
      for (int g = 0; g < 2; g++) {
        u32 out[4];
        decode_group(sm[2 * g], sm[2 * g + 1], v_group_codes(cd, t, g), (fl >> (4 * r + 2 * g)) & 3u, pos, esc,
                     b3w[2 * g], b3w[2 * g + 1], dw[2 * g], dw[2 * g + 1], out);
#pragma unroll
        for (int h = 0; h < 2; h++) {
          int w = 2 * g + h;
          uint16_t* x = &ws.xs[row * XS_STRIDE + r];
          x[8 * (4 * w)] = (uint16_t)out[2 * h]; x[8 * (4 * w + 1)] = (uint16_t)(out[2 * h] >> 16);
          x[8 * (4 * w + 2)] = (uint16_t)out[2 * h + 1]; x[8 * (4 * w + 3)] = (uint16_t)(out[2 * h + 1] >> 16);
        }
      }
    }
  }
  __syncwarp();
}

// Copy the first nvalid rows of ws.xs to a [*, 128] bf16 matrix (16-byte stores).
__device__ __forceinline__ void unstage_rows(const WarpScratch& ws, uint16_t* dst, long row_stride, int nvalid, int lane) {
#pragma unroll
  for (int k = 0; k < 8; k++) {
    int c = lane + 32 * k, row = c >> 4, col = (c & 15) * 8;
    if (row < nvalid) *reinterpret_cast<uint4*>(dst + (long)row * row_stride + col) = *reinterpret_cast<const uint4*>(&ws.xs[row * XS_STRIDE + col]);
  }
}

}  // namespace gaac
