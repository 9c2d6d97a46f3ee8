// Byte-SWAR building blocks of the GAAC tile format, shared by every kernel (encoder, decoder, fused attention).
// All functions are __host__ __device__ so the bit logic can be exercised on the CPU by the test-suite.
//
// Format facts used here (reference: gaac/codec.py:1-18,139-172; gaac/kernel.py:29-46):
//   bf16 bits x  ->  e = (x >> 7) & 0xFF,  sm = ((x >> 8) & 0x80) | (x & 0x7F)
//   group of 8 stored positions: tier 0 -> e = base3 + code, tier 1 -> e = base4 + code + 8*bit4, tier 2 -> e = code | hi5 << 3
//   tags: 2 bits per group in a u32 per row (bit0 = promoted, bit1 = raw); escape bytes: tier 1 -> 1, tier 2 -> 5.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define GAAC_HD __host__ __device__ __forceinline__
#else
#define GAAC_HD inline
#endif

namespace gaac {

typedef uint32_t u32;
typedef uint64_t u64;

constexpr int D = 128;          // head dim
constexpr int T = 16;           // tokens per tile
constexpr int CB = 48;          // code bytes per row
constexpr int TILE_SM = T * D;  // 2048
constexpr int TILE_CD = T * CB; // 768
constexpr int TILE_MAX_ESC = 1280;
constexpr int SLOT_CD_OFF = 2048, SLOT_FL_OFF = 2816, SLOT_OVF_OFF = 2880;   // paged tile slot layout (gaac/vllm/store.py:18)

// ---- portable intrinsics ---------------------------------------------------------------------------------------
GAAC_HD u32 prmt(u32 a, u32 b, u32 sel) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(a, b, sel);
#else
  u64 pool = (u64)a | ((u64)b << 32);
  u32 r = 0;
  for (int i = 0; i < 4; i++) r |= (u32)((pool >> (8 * ((sel >> (4 * i)) & 7))) & 0xFF) << (8 * i);
  return r;
#endif
}
GAAC_HD u32 funnel_r(u32 lo, u32 hi, int sh) {          // (hi:lo) >> sh, 0 <= sh < 32
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(lo, hi, sh);
#else
  return sh ? (u32)((((u64)hi << 32) | lo) >> sh) : lo;
#endif
}
GAAC_HD int popc(u32 x) {
#if defined(__CUDA_ARCH__)
  return __popc(x);
#else
  return __builtin_popcount(x);
#endif
}

// ---- tags -> escape byte counts --------------------------------------------------------------------------------
// escape bytes of a row with tag word fl (tier 1 -> 1 byte, tier 2 -> 5 bytes)                  gaac/kernel.py:46
GAAC_HD int row_esc_bytes(u32 fl) { return popc(fl & 0x55555555u) + 4 * popc(fl & 0xAAAAAAAAu); }
// escape bytes of the groups below bit position `bits` of the tag word                            gaac/kernel.py:29
GAAC_HD int esc_prefix(u32 fl, int bits) {
  u32 low = bits >= 32 ? fl : (fl & ((1u << bits) - 1u));
  return popc(low & 0x55555555u) + 4 * popc(low & 0xAAAAAAAAu);
}

// ---- decode side -----------------------------------------------------------------------------------------------
// four 3-bit codes at bits 0..11 of u (higher bits ignored) -> one code per byte
GAAC_HD u32 spread_codes4(u32 u) {
  u32 v = u & 0xFFFu;
  u32 y = (v | (v << 10)) & 0x003F003Fu;
  return (y | (y << 5)) & 0x07070707u;
}
// four 1-bit flags at bits 0..3 of n (n < 16) -> 8 * flag per byte (the 4th bit of a 4-bit window code)
GAAC_HD u32 spread_bit4(u32 n) { return (n * 0x01020408u) & 0x08080808u; }
// four 5-bit fields at bits 0..19 of u (higher bits ignored) -> field << 3 per byte (raw-tier exponent high bits)
GAAC_HD u32 spread_hi5(u32 u) {
  u32 v = u & 0xFFFFFu;
  u32 y = (v & 0x3FFu) | ((v << 6) & 0x03FF0000u);            // fields (0,1) in the low half, (2,3) in the high half
  u32 z = (y & 0x001F001Fu) | ((y << 3) & 0x1F001F00u);       // one field per byte
  return z << 3;
}
// sign/mantissa bytes (4) + exponent bytes (4) -> bf16 pairs (elements 0,1) and (2,3)             gaac/kernel.py:34-36
GAAC_HD void bf16x4(u32 sm4, u32 e4, u32& p01, u32& p23) {
  u32 h4 = (sm4 & 0x80808080u) | ((e4 >> 1) & 0x7F7F7F7Fu);
  u32 l4 = ((e4 << 7) & 0x80808080u) | (sm4 & 0x7F7F7F7Fu);
  p01 = prmt(l4, h4, 0x5140);
  p23 = prmt(l4, h4, 0x7362);
}
// 12-bit code field number s (0..7) of a 96-bit little-endian string held in c[0..2]
GAAC_HD u32 code_field12(const u32* c, int s) {
  int p = 12 * s;
  u32 lo = c[p >> 5], hi = (p >> 5) < 2 ? c[(p >> 5) + 1] : 0u;
  return funnel_r(lo, hi, p & 31);
}

// ---- encode side -----------------------------------------------------------------------------------------------
// two bf16 pairs (elements 0,1) (2,3) -> sign/mantissa bytes and exponent bytes
GAAC_HD void split_bf16x4(u32 p01, u32 p23, u32& sm4, u32& e4) {
  u32 l4 = prmt(p01, p23, 0x6420), h4 = prmt(p01, p23, 0x7531);
  sm4 = (h4 & 0x80808080u) | (l4 & 0x7F7F7F7Fu);
  e4 = ((h4 << 1) & 0xFEFEFEFEu) | ((l4 >> 7) & 0x01010101u);
}
// per-byte a - b (mod 256), no borrow across bytes
GAAC_HD u32 sub_bytes(u32 a, u32 b) {
  return ((a | 0x80808080u) - (b & 0x7F7F7F7Fu)) ^ ((a ^ ~b) & 0x80808080u);
}
// four codes (one per byte, < 8) -> 12 bits
GAAC_HD u32 pack_codes4(u32 c4) { return (c4 & 7u) | ((c4 >> 5) & 0x38u) | ((c4 >> 10) & 0x1C0u) | ((c4 >> 15) & 0xE00u); }
// bit 3 of each byte -> 4 bits
GAAC_HD u32 pack_bit4(u32 d4) { return (((d4 >> 3) & 0x01010101u) * 0x10204080u) >> 28; }
// (byte >> 3) of each byte -> 20 bits
GAAC_HD u32 pack_hi5(u32 e4) {
  u32 f = (e4 >> 3) & 0x1F1F1F1Fu;
  return (f & 0x1Fu) | ((f >> 3) & 0x3E0u) | ((f >> 6) & 0x7C00u) | ((f >> 9) & 0xF8000u);
}

// Encode one group of 8 stored positions given its exponent bytes (elements 0-3 in e_lo, 4-7 in e_hi) and the bases.
// Returns the tier tag (0, 1, 3); codes24 = 8 x 3-bit codes; esc = escape payload (1 byte for tier 1, 40 bits for tier 2).
GAAC_HD u32 encode_group(u32 e_lo, u32 e_hi, u32 b3_lo, u32 b3_hi, u32 b4_lo, u32 b4_hi, u32& codes24, u64& esc) {
  // Both windows are tried up front and the tier is picked with selects: in a warp some lane nearly always needs the 4-bit
  // window, so a branch per tier would run both paths one after the other.  Only the raw tier (under 1 %) branches.
  const u32 d3l = sub_bytes(e_lo, b3_lo), d3h = sub_bytes(e_hi, b3_hi);
  const u32 d4l = sub_bytes(e_lo, b4_lo), d4h = sub_bytes(e_hi, b4_hi);
  const bool t0 = ((d3l | d3h) & 0xF8F8F8F8u) == 0;
  const bool t1 = ((d4l | d4h) & 0xF0F0F0F0u) == 0;
  if (t0 | t1) {
    const u32 cl = t0 ? d3l : (d4l & 0x07070707u), ch = t0 ? d3h : (d4h & 0x07070707u);
    codes24 = pack_codes4(cl) | (pack_codes4(ch) << 12);
    esc = t0 ? 0u : (pack_bit4(d4l) | (pack_bit4(d4h) << 4));
    return t0 ? 0u : 1u;
  }
  codes24 = pack_codes4(e_lo & 0x07070707u) | (pack_codes4(e_hi & 0x07070707u) << 12);
  esc = (u64)pack_hi5(e_lo) | ((u64)pack_hi5(e_hi) << 20); return 3u;
}

// Rebuild the exponent bytes of one half group (4 stored positions).
//   code12: the four 3-bit codes; tag: 0/1/3; half: 0 = elements 0-3, 1 = elements 4-7 of the group;
//   esc: escape payload of the group (tier 1: one byte, tier 2: 40 bits), ignored for tier 0.
GAAC_HD u32 decode_half_group(u32 code12, u32 tag, int half, u64 esc, u32 b3w, u32 b4w) {
  u32 c4 = spread_codes4(code12);
  if (tag == 0u) return b3w + c4;
  if (tag == 1u) return b4w + c4 + spread_bit4((u32)(esc >> (4 * half)) & 0xFu);
  return c4 | spread_hi5((u32)(esc >> (20 * half)));
}

}  // namespace gaac
