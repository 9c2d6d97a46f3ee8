// Lane-level view of a GAAC tile (16 tokens x 128 channels): what one lane of a warp encodes or rebuilds.
// Everything here is lane-local and __host__ __device__; the warp-level glue (prefix sums over rows, the tag-word OR,
// staging) lives in the kernels and is emulated by a plain loop in the host-side test library.
//
// Storage order (reference: gaac/codec.py:29-67):
//   K tile = two octets of 8 tokens.  Lane l of octet o owns token 8o + (l >> 2) and, with j = l & 3, stored positions
//     [32j, 32j+32): position 32j + 4s + q  <->  channel 16s + 2j + {0,1,8,9}[q].  Its 32 sign/mantissa bytes sit at
//     o*1024 + 32l, its 12 code bytes at o*384 + 12l.  Groups of the lane: 4j + g, g = 0..3 (positions 8g..8g+7 of the lane).
//   V tile: lane l, j = l & 3, r = l >> 2 owns tokens (2j, 2j+1, 2j+8, 2j+9) and stored positions [16r, 16r+16):
//     position 16r + n  <->  channel 8n + r.  Token slot t: 16 sign/mantissa bytes at 64l + 16t, 6 code bytes at 24l + 6t.
//     Groups of the lane: 2r + g, g = 0..1.
#pragma once
#include "gaac_swar.h"

namespace gaac {

// ---- per-lane base words ---------------------------------------------------------------------------------------
// K lane j: word s = bases of channels 16s + 2j + {0,1,8,9}                                      gaac/kernel.py:70-72
GAAC_HD void k_base_words(const uint8_t* row, int j, u32 w[8]) {
  for (int s = 0; s < 8; s++) {
    int d0 = 16 * s + 2 * j;
    w[s] = (u32)row[d0] | ((u32)row[d0 + 1] << 8) | ((u32)row[d0 + 8] << 16) | ((u32)row[d0 + 9] << 24);
  }
}
// V lane class r: word w = bases of channels 8(4w + i) + r, i = 0..3                              gaac/kernel.py:73-75
GAAC_HD void v_base_words(const uint8_t* row, int r, u32 w[4]) {
  for (int i = 0; i < 4; i++)
    w[i] = (u32)row[32 * i + r] | ((u32)row[32 * i + 8 + r] << 8) | ((u32)row[32 * i + 16 + r] << 16) | ((u32)row[32 * i + 24 + r] << 24);
}

// ---- encode ----------------------------------------------------------------------------------------------------
// One lane's share of one K token row.  row: 128 bf16 bit patterns in natural channel order (any 4-byte aligned memory).
// Outputs: sm[8] (32 bytes in stored order), cd[3] (96 code bits), tags8 (2 bits x 4 groups), esc[4] (payload per group).
GAAC_HD void encode_k_lane(const uint16_t* row, int j, const u32 b3[8], const u32 b4[8], u32 sm[8], u32 cd[3], u32& tags8, u64 esc[4]) {
  u32 e[8];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int s = 0; s < 8; s++) {
    const u32* p = reinterpret_cast<const u32*>(row + 16 * s + 2 * j);
    split_bf16x4(p[0], p[4], sm[s], e[s]);
  }
  tags8 = 0;
  u32 c24[4];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int g = 0; g < 4; g++) {
    u32 tag = encode_group(e[2 * g], e[2 * g + 1], b3[2 * g], b3[2 * g + 1], b4[2 * g], b4[2 * g + 1], c24[g], esc[g]);
    tags8 |= tag << (2 * g);
  }
  cd[0] = c24[0] | (c24[1] << 24);
  cd[1] = (c24[1] >> 8) | (c24[2] << 16);
  cd[2] = (c24[2] >> 16) | (c24[3] << 8);
}

// One lane's share of one V token row (stored positions 16r .. 16r+15).  sm[4], cd48 (48 code bits), tags4, esc[2].
GAAC_HD void encode_v_lane(const uint16_t* row, int r, const u32 b3[4], const u32 b4[4], u32 sm[4], u64& cd48, u32& tags4, u64 esc[2]) {
  u32 e[4];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int w = 0; w < 4; w++) {
    u32 p01 = (u32)row[8 * (4 * w) + r] | ((u32)row[8 * (4 * w + 1) + r] << 16);
    u32 p23 = (u32)row[8 * (4 * w + 2) + r] | ((u32)row[8 * (4 * w + 3) + r] << 16);
    split_bf16x4(p01, p23, sm[w], e[w]);
  }
  tags4 = 0; cd48 = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int g = 0; g < 2; g++) {
    u32 c24;
    u32 tag = encode_group(e[2 * g], e[2 * g + 1], b3[2 * g], b3[2 * g + 1], b4[2 * g], b4[2 * g + 1], c24, esc[g]);
    tags4 |= tag << (2 * g);
    cd48 |= (u64)c24 << (24 * g);
  }
}

GAAC_HD int tag_esc_bytes(u32 tag) { return (int)(tag & 1u) + 2 * (int)(tag & 2u); }   // 0, 1, 5 for tags 0, 1, 3

// ---- decode ----------------------------------------------------------------------------------------------------
// Rebuild one group (8 stored positions = two sign/mantissa words) into four bf16x2 words.
//   sm_lo/sm_hi: sign/mantissa words of elements 0-3 / 4-7; c24: the group's 8 codes; tag: 0/1/3;
//   esc.byte(pos) / esc.bytes5(pos): escape byte / 40-bit payload at escape position pos (advanced past this group on return);
//   b3*: 3-bit-window base words of the two half groups, d*: (4-bit-window base word - 3-bit-window base word) as a plain
//   32-bit difference, so b3 + 1*d is the 4-bit base word exactly.  Tier 0/1 is branch-free; the raw tier patches the addend.
template <class Esc>
GAAC_HD void decode_group(u32 sm_lo, u32 sm_hi, u32 c24, u32 tag, int& pos, const Esc& esc,
                          u32 b3lo, u32 b3hi, u32 dlo, u32 dhi, u32 out[4]) {
  const u32 m1 = tag & 1u;
  u32 xe = 0u;
  if (tag == 1u) xe = esc.byte(pos);
  u32 x0 = spread_bit4(xe & 0xFu), x1 = spread_bit4(xe >> 4);
  const u32 blo = b3lo + m1 * dlo, bhi = b3hi + m1 * dhi;
  if (tag & 2u) {                                   // raw exponents: e = code | hi5 << 3 (the base must not contribute)
    u64 w = esc.bytes5(pos);
    x0 = spread_hi5((u32)w) - blo;
    x1 = spread_hi5((u32)(w >> 20)) - bhi;
  }
  pos += tag_esc_bytes(tag);
  u32 e0 = spread_codes4(c24) + blo + x0;
  u32 e1 = spread_codes4(c24 >> 12) + bhi + x1;
  bf16x4(sm_lo, e0, out[0], out[1]);
  bf16x4(sm_hi, e1, out[2], out[3]);
}

// Table-driven variant of decode_group for the fused attention kernel (fewer ALU instructions, no branch for the 4-bit window):
//   lutx[b] = { spread_bit4(b & 15), spread_bit4(b >> 4) } for every escape byte value b (2 KiB, shared memory);
//   esc: base of the tile's escape bytes (any address space), zero: address of a zero byte read by groups without an escape byte;
//   bw = { b3lo, b3hi, dlo, dhi } base words of the group as in decode_group.
// The raw tier (rare) is a divergent branch that reads its five bytes as two aligned words.
struct u32x4 { u32 x, y, z, w; };
struct u32x2 { u32 x, y; };
GAAC_HD void fill_lutx(u32x2* lutx, int i) { lutx[i].x = spread_bit4((u32)i & 0xFu); lutx[i].y = spread_bit4((u32)i >> 4); }
GAAC_HD void decode_group_lut(u32 sm_lo, u32 sm_hi, u32 c24, u32 tag, int& pos, const uint8_t* esc, const uint8_t* zero,
                              const u32x2* lutx, const u32x4& bw, u32 out[4]) {
  const u32 m1 = tag & 1u;
  const uint8_t* pe = (tag == 1u) ? esc + pos : zero;
  const u32x2 x = lutx[*pe];
  u32 x0 = x.x, x1 = x.y;
  const u32 blo = bw.x + m1 * bw.z, bhi = bw.y + m1 * bw.w;
  if (tag & 2u) {                                   // raw exponents: e = code | hi5 << 3 (the base must not contribute)
    const uint8_t* p = esc + pos;
    const int sh = 8 * (int)(reinterpret_cast<uintptr_t>(p) & 3);
    const u32* a = reinterpret_cast<const u32*>(reinterpret_cast<uintptr_t>(p) & ~(uintptr_t)3);
    const u32 w0 = a[0], w1 = a[1];                                           // five bytes at offset <= 3 never leave two words
    const u32 lo = funnel_r(w0, w1, sh), hi = w1 >> sh;                       // bytes 0-3 and byte 4 of the group's payload
    x0 = spread_hi5(lo) - blo;
    x1 = spread_hi5(funnel_r(lo, hi, 20)) - bhi;
    pos += 4;
  }
  pos += (int)m1;
  const u32 e0 = spread_codes4(c24) + blo + x0;
  const u32 e1 = spread_codes4(c24 >> 12) + bhi + x1;
  bf16x4(sm_lo, e0, out[0], out[1]);
  bf16x4(sm_hi, e1, out[2], out[3]);
}

// 24 code bits of group g (0..3) of a K lane (96-bit string in cd[0..2])
GAAC_HD u32 k_group_codes(const u32 cd[3], int g) {
  switch (g) {
    case 0: return cd[0];
    case 1: return funnel_r(cd[0], cd[1], 24);
    case 2: return funnel_r(cd[1], cd[2], 16);
    default: return cd[2] >> 8;
  }
}
// 24 code bits of group g (0..1) of token slot t (0..3) of a V lane (192-bit string in cd[0..5])
GAAC_HD u32 v_group_codes(const u32 cd[6], int t, int g) {
  int p = 48 * t + 24 * g;            // bit offset: multiples of 24
  int w = p >> 5, sh = p & 31;
  u32 hi = w < 5 ? cd[w + 1] : 0u;
  return funnel_r(cd[w], hi, sh);
}

}  // namespace gaac
