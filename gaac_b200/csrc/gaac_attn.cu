// Fused decode attention over GAAC-compressed K/V (sm_100a): slot layout and paged layout in one kernel template.
//
// CTA = (batch row, kv head, context split), ATT_WARPS warps, one CTA per SM.  Every warp streams its own 16-token tiles
// through a private two-stage shared-memory ring filled by bulk asynchronous copies (the TMA engine without a tensor map,
// completion counted in bytes on an mbarrier), rebuilds BF16 K/V fragments in registers (byte-SWAR, gaac_tile.h) and feeds
// mma.sync m16n8k16:
//   S^T[16 tok x 8 heads] = K[16 x 128] . Q^T        O^T[128 dims x 8 heads] += V^T[128 x 16 tok] . P^T
// with an fp32 online softmax in the exp2 domain whose maximum is raised lazily.  Raw BF16 tiles (the slot layout's tail, the
// paged layout's filling block and raw-fallback tiles) are read straight from global memory into the same fragments.  Tiles
// are handed to the warps of a CTA from a shared counter.  The warps of a CTA are merged in shared memory, the CTA writes
// one partial (m, l, acc[128]) per query head, and the last CTA of a (row, kv head) to finish merges the splits and writes
// the output, so one launch does the whole layer.
//
// What the measurements on B200 say (they shaped the code below):
//  * per-lane cp.async copies (18 instructions per tile pair and warp) kept the load/store unit 60 % busy, and it is shared
//    with the fragment reads: the L1-bypassing form sends one sector request per lane and writes shared memory one lane
//    chunk per wavefront, the caching form coalesces but still costs ~22 cycles per instruction.  Bulk copies take that
//    work off the SM; they want few large copies (one 128-byte copy per row, which would allow a conflict-free skewed
//    layout, was 15 % slower), so shared memory holds the storage order and the 16-byte fragment reads accept a 2-way (K) /
//    4-way (V) bank conflict (worth 0.7 us of 74).
//  * the kernel is bound by instruction issue (ALU pipe) and by the shared-memory pipe, not by HBM: spreading the 3-bit
//    codes through a 4096-entry table costs one load with ~3.5-way bank conflicts, by arithmetic two multiply-adds and
//    three logic instructions.  Which is faster moved with the rest of the kernel (table while the copies loaded the
//    load/store unit less than the integer pipe, half and half after the bulk copies brought the storage-order conflicts);
//    in the final kernel arithmetic only is fastest by 1 %, table only slowest by 4 % (GAAC_LUTC = 0 / 2 / 1).
//
// Fragment conventions follow the reference kernel (gaac/kernel.py:62-66,160-194), whose storage order they mirror.
#include <cuda_bf16.h>
#include <math_constants.h>
#include <algorithm>
#include "gaac_api.cuh"
#include "gaac_tile.h"

namespace gaac {

#ifndef GAAC_LUTC
#define GAAC_LUTC 0
#endif
// Softmax weights enter the PV product as BF16 (tensor-core operand).  GAAC_SPLIT_P = 1: each weight goes in as the sum of two
// BF16 numbers, its rounded value and the rounded remainder (two MMAs on the same V fragments), which brings the relative error
// of a weight from 2^-8 down to 2^-16; = 0: the rounded value only, as the reference kernel does (gaac/kernel.py:178).
#ifndef GAAC_SPLIT_P
#define GAAC_SPLIT_P 1
#endif
// Build-time knobs of the experiments that shaped the kernel (the defaults are what ships):
//   GAAC_WARPS    warps per CTA (one CTA per SM; the register budget per thread follows from it).  Only 16 is tested for results;
//                 12 and 18 were timing experiments, 8 is known to give wrong output
//   GAAC_ESC_WIN  escape bytes staged per tile and kind
//   GAAC_QSMEM    1: the query fragments live in a shared-memory table read once per K group instead of 16 registers per lane
#ifndef GAAC_WARPS
#define GAAC_WARPS 16
#endif
#ifndef GAAC_ESC_WIN
#define GAAC_ESC_WIN 256
#endif
#ifndef GAAC_QSMEM
#define GAAC_QSMEM 0
#endif
//   GAAC_ALU2FMA  bit mask of integer operations of the group decoder written as multiply-adds, which issue on the FMA pipe
//                 instead of the half-rate ALU pipe: 1 = the >> 12 of the code word as a high multiply, 2 = the three-term
//                 exponent sum as two multiply-adds by 1, 4 = the escape position advance as a multiply-add by 1
#ifndef GAAC_ALU2FMA
#define GAAC_ALU2FMA 0
#endif
//   GAAC_ABLATE   timing-only builds that compute WRONG results, to see where the time goes: 1 = no rebuild at all (fragments
//                 taken from the staged bytes as they are), 2 = every group decoded as tier 0 (no tags, no escape bytes),
//                 3 = raw tier compiled out
#ifndef GAAC_ABLATE
#define GAAC_ABLATE 0
#endif
//   GAAC_RAWPATCH 1: raw-tier groups are resolved by a short pass per tile that turns each of them into a table entry, after
//                 which the group decoder has no branch at all; 0: the decoder branches on the raw tag of every group
#ifndef GAAC_RAWPATCH
#define GAAC_RAWPATCH 1
#endif
//   GAAC_DEEP     1: a warp's copies run a whole tile ahead: the stage it has just consumed is refilled at once with the tile after
//                 the next one; 0: the next tile's copies are issued in the middle of the current tile (half a tile ahead).
//                 Measured 2 % SLOWER at 1 (with and without the rebuild): the copies already arrive in time, the kernel waits
//                 for instruction issue, not for memory
#ifndef GAAC_DEEP
#define GAAC_DEEP 0
#endif
constexpr int ATT_WARPS = GAAC_WARPS;
constexpr int ATT_THREADS = ATT_WARPS * 32;
constexpr int NSTAGE = 2;
constexpr int ESC_WIN = GAAC_ESC_WIN;                       // escape bytes staged per tile and kind; longer tiles read theirs from global memory
// ---- stage layout (bytes)
// Stage = 16 bytes (mbarrier, then 8 bytes that stay zero) + a block per side:
//   sign/mantissa (2048, storage order) | codes (768) | tag words (64) | escape window (ESC_WIN + 16: it starts at the
//   16-byte boundary below the tile's first escape byte).  Every piece is ONE bulk copy: copies of 128 bytes (one per
//   row, skewed to avoid the bank conflicts of the storage order) were measured 15 % slower, the copy engine wants few large
//   copies, so the fragment reads accept a 2-way (K) / 4-way (V) conflict.
// A side block is laid out as the paged tile slot is, so the paged layout fetches a whole slot with one copy.
constexpr int ESC_COPY = ESC_WIN + 16;
constexpr int SM_ROW = 128;
constexpr int SB_SM = 0, SB_CD = SB_SM + 16 * SM_ROW, SB_FL = SB_CD + 768, SB_ESC = SB_FL + 64, SIDE_BYTES = SB_ESC + ESC_COPY;
constexpr int ST_MBAR = 0, ST_ZERO = 8, ST_K = 16, ST_V = ST_K + SIDE_BYTES;
constexpr int ST_KSM = ST_K + SB_SM, ST_KCD = ST_K + SB_CD, ST_KFL = ST_K + SB_FL, ST_KESC = ST_K + SB_ESC;
constexpr int ST_VSM = ST_V + SB_SM, ST_VCD = ST_V + SB_CD, ST_VFL = ST_V + SB_FL, ST_VESC = ST_V + SB_ESC;
constexpr int STAGE_BYTES = ST_V + SIDE_BYTES;
static_assert(SB_CD - SB_SM == SLOT_CD_OFF && SB_FL - SB_SM == SLOT_FL_OFF && SB_ESC - SB_SM == SLOT_OVF_OFF, "side block laid out as the paged tile slot");
constexpr int META_TILES = 512;                      // tiles of a CTA's range whose metadata is staged (longer ranges read the rest from global)
// CTA tables: escape-byte table (2 KiB), K / V base words, per-tile metadata, and the code table: four 3-bit codes -> four bytes
// for all 4096 values of a 12-bit field (16 KiB).  The table turns four logic instructions per lookup into one shared-memory load.
constexpr int TB_LUTX = 0, TB_KB = 2048, TB_VB = TB_KB + 256, TB_META = TB_VB + 256, TB_LUTC = TB_META + 2 * META_TILES * 4;
constexpr int TB_Q = TB_LUTC + (GAAC_LUTC ? 4096 * 4 : 0);          // query fragments: [4 K groups][32 lanes] x 16 bytes
constexpr int TABLE_BYTES = TB_Q + (GAAC_QSMEM ? 4 * 32 * 16 : 0);
// Raw-tier patch table of a warp: per side PATCH_MAX entries of 8 bytes = the two exponent addends of a raw group with the
// 4-bit-window base already taken off (the decoder adds that base to every promoted group).  Tiles with more raw groups on a
// side (random bit patterns) take the decoder that branches.
constexpr int PATCH_MAX = 32, PATCH_BYTES = 2 * PATCH_MAX * 8;
constexpr int WARP_SMEM = NSTAGE * STAGE_BYTES + PATCH_BYTES;
constexpr int ATT_SMEM = TABLE_BYTES + ATT_WARPS * WARP_SMEM;
static_assert(TABLE_BYTES % 16 == 0 && STAGE_BYTES % 16 == 0 && ST_KSM % 16 == 0 && ST_KCD % 16 == 0 && ST_KFL % 16 == 0 && ST_KESC % 16 == 0 &&
              ST_VSM % 16 == 0 && ST_VCD % 16 == 0 && ST_VFL % 16 == 0 && ST_VESC % 16 == 0 && ESC_COPY % 16 == 0 && ST_MBAR % 8 == 0 && SM_ROW % 16 == 0,
              "bulk copies need 16-byte aligned shared-memory destinations and sizes");
static_assert(ATT_SMEM + 64 <= 232448, "one CTA per SM: at most 227 KB of shared memory, static part included");
static_assert(ATT_THREADS / 128 * 2 >= 8, "the fused exchange keeps at most two merged heads per thread");
constexpr unsigned FULLM = 0xffffffffu;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

struct AttnParams {
  // slot layout
  gaac_side K, V;
  const int* slot; const int* seq_len; const int* tail_len; int tail_cap; long S_pad; int n_base_rows;
  int S_uniform;                 // tokens of every cache head when seq_len == NULL (slot == NULL: batch row b reads slot b)
  // paged layout
  const uint8_t* buf; const uint16_t* raw; const int* mt; const int* bt; long bt_stride; int TS; int ovf_slot;
  const uint8_t *b3k, *b4k, *b3v, *b4v;
  // common
  const uint16_t* q; int B, n_q, n_kv, G; float scale_log2; int nsplit;
  int* counters; int* err; float* pm; float* pl; float* pa;     // err: set to 1 when a bounded wait inside the kernel ran out
  uint16_t* out; float* out_f32; float* part;
  // cross-GPU exchange (x_recv == NULL: unused): the partial of every query head is stored into every rank's receive
  // buffer, then this rank's arrival flag of the (row, kv head) group on every rank is set to the exchange number; with
  // x_fused the same CTA then waits (bounded) for the other ranks' flags, merges all ranks' rows and writes the output
  const int2* row_order;                            // paged layout, optional: {batch row, its token count}, longest row first
  int2* order_buf;                                  // room for B entries of it in the workspace
  unsigned long long* const* x_recv; int* x_epoch; int* x_ticket; int* x_err; int x_rank, x_world, x_rows_cap, x_fused;
  // debug instantiation only: the rebuilt BF16 K / V rows are written to [B*n_kv, dump_S, 128] (row = token of the head)
  uint16_t* dump_k; uint16_t* dump_v; long dump_S;
};

#ifndef GAAC_MMA_VOLATILE
#define GAAC_MMA_VOLATILE 1
#endif
#if GAAC_MMA_VOLATILE
#define GAAC_MMA_ASM asm volatile
#else
#define GAAC_MMA_ASM asm
#endif
__device__ __forceinline__ void mma16816(float* c, const u32* a, u32 b0, u32 b1) {
  GAAC_MMA_ASM("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// ---- bulk asynchronous copies (TMA engine, no tensor map): global -> shared, completion counted in bytes on an mbarrier.
// Both addresses are 16-byte aligned and the size is a multiple of 16 at every call site.
__device__ __forceinline__ void mbar_init(u32 mbar, u32 count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(u32 mbar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_add_tx(u32 mbar, u32 bytes) { asm volatile("mbarrier.expect_tx.shared::cta.b64 [%0], %1;\n" ::"r"(mbar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(u32 mbar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(mbar) : "memory"); }
__device__ __forceinline__ void bulk_g2s(u32 dst, const void* src, u32 bytes, u32 mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes), "r"(mbar) : "memory");
}
// Bounded wait for a phase of the barrier: false when it gave up (the copies of a stage normally land within microseconds;
// the bound is there so that a lost copy can never hang the GPU).
constexpr int MBAR_WAIT_LIMIT = 1 << 22;
__device__ __forceinline__ bool mbar_wait(u32 mbar, u32 parity) {
  for (int it = 0; it < MBAR_WAIT_LIMIT; it++) {
    u32 ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ float fast_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// What a warp remembers of a tile between issuing its copies and consuming it.  Slot layout: offsets of the tile's escape
// bytes inside the head's escape bytes.  Paged layout: the mode-table entries (>= 0: compressed slot, < 0: bit-complement
// of a raw tile of the pool).
struct TileMeta { int mk, mv; };

// Per-head values of the slot layout that the copy addressing needs.
struct LaneAddr {
  int ohk, ohv;                  // first escape byte of the head inside ovf
  int availk, availv;            // bytes from there to the end of the allocation (clamped to int)
};

// Running state of one warp.
struct WarpAcc {
  float acc[8][4];       // m-tile mt: c0 = O[dim 16mt+r][head 2j], c1 = [..][2j+1], c2 = O[16mt+r+8][2j], c3 = [..][2j+1]
  float m0, m1, l0, l1;  // heads 2j, 2j+1 (exp2 domain); l summed over this lane's tokens only
};

// Online softmax on the score fragment + P^T B-fragments for the PV product.
// The running maximum is only raised (and the accumulators rescaled) when some score of the tile exceeds it by more than
// RESCALE_TAU in the exp2 domain; otherwise the tile is weighted against the stale maximum, so P stays below 2^RESCALE_TAU.
// Sums and accumulators are fp32 and P keeps its relative BF16 rounding, so the result is as exact as with the true
// maximum, and the common tile needs no cross-lane reduction, no rescale factor and no accumulator multiply.
constexpr float RESCALE_TAU = 16.f;
// P^T B-fragments of one tile for the PV product: hi = the weights rounded to BF16, lo = the BF16-rounded remainders.
struct PFrag { u32 hi0, hi1, lo0, lo1; };
template <bool FULL_TILE>
__device__ __forceinline__ void softmax_step(WarpAcc& A, const float* sc, float scale_log2, int nvalid, int lane, PFrag& P) {
  const int j = lane & 3, r = lane >> 2;
  const bool v0 = FULL_TILE || r < nvalid, v8 = FULL_TILE || r + 8 < nvalid;     // a full tile needs no token masks
  const float s00 = v0 ? sc[0] * scale_log2 : -CUDART_INF_F, s01 = v0 ? sc[1] * scale_log2 : -CUDART_INF_F;
  const float s80 = v8 ? sc[2] * scale_log2 : -CUDART_INF_F, s81 = v8 ? sc[3] * scale_log2 : -CUDART_INF_F;
  float mt0 = fmaxf(s00, s80), mt1 = fmaxf(s01, s81);
  if (__any_sync(FULLM, mt0 > A.m0 + RESCALE_TAU || mt1 > A.m1 + RESCALE_TAU)) {
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) { mt0 = fmaxf(mt0, __shfl_xor_sync(FULLM, mt0, o)); mt1 = fmaxf(mt1, __shfl_xor_sync(FULLM, mt1, o)); }
    const float mn0 = fmaxf(A.m0, mt0), mn1 = fmaxf(A.m1, mt1);
    const float al0 = (mn0 == -CUDART_INF_F) ? 0.f : fast_exp2(A.m0 - mn0), al1 = (mn1 == -CUDART_INF_F) ? 0.f : fast_exp2(A.m1 - mn1);
    A.l0 *= al0; A.l1 *= al1; A.m0 = mn0; A.m1 = mn1;
#pragma unroll
    for (int n = 0; n < 8; n++) { A.acc[n][0] *= al0; A.acc[n][2] *= al0; A.acc[n][1] *= al1; A.acc[n][3] *= al1; }
  }
  const float mu0 = fmaxf(A.m0, -1e30f), mu1 = fmaxf(A.m1, -1e30f);       // a maximum of -inf (nothing seen yet) must not produce inf - inf
  const float p00 = fast_exp2(s00 - mu0), p80 = fast_exp2(s80 - mu0), p01 = fast_exp2(s01 - mu1), p81 = fast_exp2(s81 - mu1);
  A.l0 += p00 + p80; A.l1 += p01 + p81;
  // this lane publishes W0 = (P[tok r][2j], P[tok r][2j+1]), W8 = (P[tok r+8][2j], P[tok r+8][2j+1]);
  // it needs b0 = (P[tok 2j][head r], P[tok 2j+1][head r]), b1 = the same for tokens 2j+8, 2j+9
  __nv_bfloat162 x = __floats2bfloat162_rn(p00, p01), y = __floats2bfloat162_rn(p80, p81);
  const u32 W0 = *reinterpret_cast<u32*>(&x), W8 = *reinterpret_cast<u32*>(&y);
  const int srcA = 8 * j + (r >> 1), srcB = srcA + 4;
  const u32 a0 = __shfl_sync(FULLM, W0, srcA), a8 = __shfl_sync(FULLM, W8, srcA), b0w = __shfl_sync(FULLM, W0, srcB), b8w = __shfl_sync(FULLM, W8, srcB);
  const u32 sel = (r & 1) ? 0x7632u : 0x5410u;
  P.hi0 = prmt(a0, b0w, sel); P.hi1 = prmt(a8, b8w, sel);
#if GAAC_SPLIT_P
  // what the rounding dropped, exactly (p - bf16(p) is representable in fp32), rounded to BF16 in turn and routed the same way
  __nv_bfloat162 xl = __floats2bfloat162_rn(p00 - __uint_as_float(W0 << 16), p01 - __uint_as_float(W0 & 0xFFFF0000u));
  __nv_bfloat162 yl = __floats2bfloat162_rn(p80 - __uint_as_float(W8 << 16), p81 - __uint_as_float(W8 & 0xFFFF0000u));
  const u32 L0 = *reinterpret_cast<u32*>(&xl), L8 = *reinterpret_cast<u32*>(&yl);
  const u32 c0 = __shfl_sync(FULLM, L0, srcA), c8 = __shfl_sync(FULLM, L8, srcA), d0w = __shfl_sync(FULLM, L0, srcB), d8w = __shfl_sync(FULLM, L8, srcB);
  P.lo0 = prmt(c0, d0w, sel); P.lo1 = prmt(c8, d8w, sel);
#else
  P.lo0 = P.lo1 = 0u;
#endif
}

// PV for one pair of V words: tokens (2j, 2j+1, 2j+8, 2j+9) x elements (4w .. 4w+3).
__device__ __forceinline__ void pv_words(WarpAcc& A, int w, const u32 (&u01)[4], const u32 (&u23)[4], const PFrag& P) {
#if GAAC_SPLIT_P && defined(GAAC_PV_INTERLEAVE)
  // the two MMAs into one accumulator depend on each other: issue the two independent ones in between
  u32 a[4], c[4];
  a[0] = prmt(u01[0], u01[1], 0x5410); a[2] = prmt(u01[2], u01[3], 0x5410);     // dim 8(4w)+r
  a[1] = prmt(u01[0], u01[1], 0x7632); a[3] = prmt(u01[2], u01[3], 0x7632);     // dim 8(4w+1)+r
  c[0] = prmt(u23[0], u23[1], 0x5410); c[2] = prmt(u23[2], u23[3], 0x5410);     // dim 8(4w+2)+r
  c[1] = prmt(u23[0], u23[1], 0x7632); c[3] = prmt(u23[2], u23[3], 0x7632);     // dim 8(4w+3)+r
  mma16816(A.acc[2 * w], a, P.hi0, P.hi1);
  mma16816(A.acc[2 * w + 1], c, P.hi0, P.hi1);
  mma16816(A.acc[2 * w], a, P.lo0, P.lo1);
  mma16816(A.acc[2 * w + 1], c, P.lo0, P.lo1);
#else
  u32 a[4];
  a[0] = prmt(u01[0], u01[1], 0x5410); a[2] = prmt(u01[2], u01[3], 0x5410);     // dim 8(4w)+r
  a[1] = prmt(u01[0], u01[1], 0x7632); a[3] = prmt(u01[2], u01[3], 0x7632);     // dim 8(4w+1)+r
  mma16816(A.acc[2 * w], a, P.hi0, P.hi1);
#if GAAC_SPLIT_P
  mma16816(A.acc[2 * w], a, P.lo0, P.lo1);
#endif
  a[0] = prmt(u23[0], u23[1], 0x5410); a[2] = prmt(u23[2], u23[3], 0x5410);     // dim 8(4w+2)+r
  a[1] = prmt(u23[0], u23[1], 0x7632); a[3] = prmt(u23[2], u23[3], 0x7632);     // dim 8(4w+3)+r
  mma16816(A.acc[2 * w + 1], a, P.hi0, P.hi1);
#if GAAC_SPLIT_P
  mma16816(A.acc[2 * w + 1], a, P.lo0, P.lo1);
#endif
#endif
}

// rowoff / total as scan_rows leaves them: escape bytes (low half) and raw groups (high half) before the row, or of the tile
__device__ __forceinline__ int esc_part(int v) { return v & 0xFFFF; }
__device__ __forceinline__ int raw_part(int v) { return v >> 16; }

// Q^T B-fragments of the score product.  Lane (j, r) holds, for k-step s, the words q[head r][16s + 2j, +1] and
// q[head r][16s + 2j + 8, +9]; K group g of a lane uses k-steps 2g and 2g + 1.
#if GAAC_QSMEM
struct QFrag {
  const uint4* tab;                                   // [4][32] in shared memory, built once per CTA
  __device__ __forceinline__ void group(int g, int lane, u32 (&b)[4]) const { const uint4 v = tab[g * 32 + lane]; b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w; }
};
#else
struct QFrag {
  u32 qa[8][2];
  __device__ __forceinline__ void group(int g, int, u32 (&b)[4]) const { b[0] = qa[2 * g][0]; b[1] = qa[2 * g][1]; b[2] = qa[2 * g + 1][0]; b[3] = qa[2 * g + 1][1]; }
};
#endif

// Escape bytes of one tile as read by the group decoder.
//   staged window (WIN): zp = shared-memory address of a zero byte below the tile's first escape byte; a group without an
//     escape byte reads zp[0] and a 4-bit-window group reads zp[off + pos]: one multiply-add, no branch.
//   global memory (!WIN, tiles whose escapes exceed the window): plain loads at glob[pos].
//   off = distance from zp to the tile's first escape byte (the zero byte a group without escapes reads sits at zp[0]).
template <bool WIN> struct EscSrc { const uint8_t* zp; const uint8_t* glob; int off; };

// ---- byte-SWAR pieces written for the pipes of the SM: logic ops (LOP3 / PRMT / SHF) run on the ALU pipe, whose rate is half
// the issue rate, so shifts that can be merged with an add are written as multiply-adds (FMA pipe) and the 3-bit -> byte
// spreading of the codes is a table lookup (load/store pipe).
template <u32 K> __device__ __forceinline__ u32 mad_k(u32 a, u32 c) {
  u32 d; asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "n"(K), "r"(c)); return d;
}
__device__ __forceinline__ void bf16x4_dev(u32 sm4, u32 e4, u32& p01, u32& p23) {
  const u32 eh = __umulhi(e4, 0x80000000u);                          // e4 >> 1
  const u32 el = mad_k<128u>(e4, 0u);                                // e4 << 7
  const u32 h4 = (sm4 & 0x80808080u) | (eh & 0x7F7F7F7Fu);
  const u32 l4 = (el & 0x80808080u) | (sm4 & 0x7F7F7F7Fu);
  p01 = prmt(l4, h4, 0x5140); p23 = prmt(l4, h4, 0x7362);
}
// four 5-bit fields at bits 0..19 of u -> field << 3 per byte (raw-tier exponent high bits); same result as spread_hi5
__device__ __forceinline__ u32 spread_hi5_dev(u32 u) {
  const u32 y = mad_k<64u>(u & 0xFFC00u, u & 0x3FFu);               // fields 0,1 at bits 0-9, fields 2,3 at bits 16-25
  return mad_k<64u>(y & 0x03E003E0u, (y & 0x001F001Fu) << 3);       // odd fields up 3 more bits, everything << 3
}

// Rebuild one group (two sign/mantissa words) into four bf16x2 words.  Same results as decode_group_lut (gaac_tile.h);
// pos16 = es.off + escape position of the group, advanced past it on return; lutc = the 4096-entry code table.
// RT (only with WIN): raw groups were turned into patch-table entries by build_raw_patches, which also left each entry's number in
// the first payload byte of its group: the addends of EVERY group then come from one load, out of the escape-byte table
// (byte = the 4-bit-window escape byte, or the zero byte) or out of the patch table (byte = entry number), chosen by address
// arithmetic, and the decoder has no branch.  patch_rel = patch table address - escape-byte table address (shared memory).
template <bool WIN, bool RT>
__device__ __forceinline__ void decode_group_dev(u32 sm_lo, u32 sm_hi, u32 c24, u32 tg, int& pos16, const EscSrc<WIN>& es,
                                                 const u32x2* lutx, const uint8_t* lutc, const u32x4& bw, u32 out[4], u32 patch_rel = 0u) {
  static_assert(WIN || !RT, "the patch table goes with the staged escape window");
  const u32 m1 = tg & 1u;                             // promoted (tags are 0, 1 or 3)
  u32 xe;
  if (WIN) xe = es.zp[m1 * (u32)pos16];               // raw groups read a payload byte here; their addends are replaced below
  else xe = m1 ? es.glob[pos16 - es.off] : 0u;
  u32 x0, x1;
  if (RT) {
    const u32 r2 = tg & 2u;                           // 2 for a raw group
    const u32x2 x = *reinterpret_cast<const u32x2*>(reinterpret_cast<const uint8_t*>(lutx) + (8u * xe + r2 * (patch_rel >> 1)));
    x0 = x.x; x1 = x.y;
    pos16 += (int)(2u * r2);                          // a raw payload is five bytes: four here, one below with every promoted group
  } else {
    const u32x2 x = lutx[xe];
    x0 = x.x; x1 = x.y;
  }
#if GAAC_LUTC == 1
  const u32 c_lo = *reinterpret_cast<const u32*>(lutc + ((c24 << 2) & 0x3FFCu));
  const u32 c_hi = *reinterpret_cast<const u32*>(lutc + ((c24 >> 10) & 0x3FFCu));
#elif GAAC_LUTC == 2
  // one half through the table (load/store pipe), the other half by arithmetic (ALU + FMA pipes): balances the pipes
  const u32 c_lo = *reinterpret_cast<const u32*>(lutc + ((c24 << 2) & 0x3FFCu));
  const u32 th = (c24 >> 12) & 0xFFFu;
  const u32 xh = mad_k<1023u>((c24 >> 12) & 0xFC0u, th);
  const u32 c_hi = mad_k<31u>(xh & 0x00380038u, xh);
#else
  // four 3-bit codes -> four bytes in two steps; each step moves the upper fields with a multiply-add: (t & M) * (2^k - 1) + t
#if GAAC_ALU2FMA & 1
  const u32 c12 = __umulhi(c24, 1u << 20);            // c24 >> 12
#else
  const u32 c12 = c24 >> 12;
#endif
  const u32 tl = c24 & 0xFFFu, th = c12 & 0xFFFu;
  const u32 xl = mad_k<1023u>(c24 & 0xFC0u, tl), xh = mad_k<1023u>(c12 & 0xFC0u, th);
  const u32 c_lo = mad_k<31u>(xl & 0x00380038u, xl), c_hi = mad_k<31u>(xh & 0x00380038u, xh);
#endif
  const u32 blo = bw.x + m1 * bw.z, bhi = bw.y + m1 * bw.w;
#if GAAC_ABLATE == 3
  if (false) {
#else
  if (!RT && (tg & 2u)) {                             // raw exponents: e = code | hi5 << 3 (the base must not contribute)
#endif
    u32 w0, w1; int sh;
    if (WIN) {
      const u32 a = (u32)__cvta_generic_to_shared(es.zp) + (u32)pos16;
      sh = 8 * (int)(a & 3u);
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w0) : "r"(a & ~3u) : "memory");
      asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(w1) : "r"(a & ~3u) : "memory");
    } else {
      const uint8_t* p = es.glob + (pos16 - es.off);
      sh = 8 * (int)(reinterpret_cast<uintptr_t>(p) & 3);
      const u32* a = reinterpret_cast<const u32*>(reinterpret_cast<uintptr_t>(p) & ~(uintptr_t)3);
      w0 = a[0]; w1 = a[1];
    }
    const u32 lo = funnel_r(w0, w1, sh), hi = w1 >> sh;              // bytes 0-3 and byte 4 of the payload
    x0 = spread_hi5_dev(lo & 0xFFFFFu) - blo;
    x1 = spread_hi5_dev(funnel_r(lo, hi, 20) & 0xFFFFFu) - bhi;
    pos16 += 4;
  }
#if GAAC_ALU2FMA & 4
  pos16 = (int)mad_k<1u>(m1, (u32)pos16);
#else
  pos16 += (int)m1;
#endif
#if GAAC_ALU2FMA & 2
  bf16x4_dev(sm_lo, mad_k<1u>(c_lo, mad_k<1u>(blo, x0)), out[0], out[1]);
  bf16x4_dev(sm_hi, mad_k<1u>(c_hi, mad_k<1u>(bhi, x1)), out[2], out[3]);
#else
  bf16x4_dev(sm_lo, c_lo + blo + x0, out[0], out[1]);
  bf16x4_dev(sm_hi, c_hi + bhi + x1, out[2], out[3]);
#endif
}

// Scores of one compressed K tile: sc += K . Q^T.  flrow / rowoff: tag word and escape offset of row (lane & 15) held by
// lanes 0-15.
// dump (debug instantiation only): where token 0 of this tile goes in the [token][128] dump of the head; every lane writes the
// fragment words it rebuilt at the (token, channel) pairs they stand for, rows >= nvalid are left alone.
template <bool WIN, bool DUMP, bool RT = false>
__device__ __forceinline__ void k_scores(float* sc, const uint8_t* stage, const uint8_t* tables, const EscSrc<WIN>& es, u32 flrow, int rowoff,
                                         int lane, const QFrag& Q, uint16_t* dump = nullptr, int nvalid = T, u32 patch_rel = 0u) {
  const int j = lane & 3, r = lane >> 2;
  const u32x2* lutx = reinterpret_cast<const u32x2*>(tables + TB_LUTX);
  u32 t8[2]; int pos[2]; uint4 s0[2], s1[2]; u32 cd[2][3];
  float s2[4] = {0.f, 0.f, 0.f, 0.f};                  // second accumulator: two dependent MMA chains of four instead of one of eight
#pragma unroll
  for (int o = 0; o < 2; o++) {
    const u32 fl = __shfl_sync(FULLM, flrow, 8 * o + r);
    pos[o] = esc_part(__shfl_sync(FULLM, rowoff, 8 * o + r)) + esc_prefix(fl, 8 * j) + es.off;
    t8[o] = fl >> (8 * j);
    s0[o] = *reinterpret_cast<const uint4*>(stage + ST_KSM + (8 * o + (lane >> 2)) * SM_ROW + 32 * (lane & 3));   // storage order, skewed rows
    s1[o] = *reinterpret_cast<const uint4*>(stage + ST_KSM + (8 * o + (lane >> 2)) * SM_ROW + 32 * (lane & 3) + 16);
    const u32* c = reinterpret_cast<const u32*>(stage + ST_KCD + o * 384 + 12 * lane);
    cd[o][0] = c[0]; cd[o][1] = c[1]; cd[o][2] = c[2];
  }
#pragma unroll
  for (int g = 0; g < 4; g++) {
    const u32x4 bw = *reinterpret_cast<const u32x4*>(tables + TB_KB + 16 * (4 * j + g));
    u32 f[2][4];
#pragma unroll
    for (int o = 0; o < 2; o++) {
      const u32 smlo = g == 0 ? s0[o].x : g == 1 ? s0[o].z : g == 2 ? s1[o].x : s1[o].z;
      const u32 smhi = g == 0 ? s0[o].y : g == 1 ? s0[o].w : g == 2 ? s1[o].y : s1[o].w;
#if GAAC_ABLATE == 1
      f[o][0] = smlo; f[o][1] = smhi; f[o][2] = smlo ^ cd[o][0]; f[o][3] = smhi ^ cd[o][g % 3];
#elif GAAC_ABLATE == 2
      decode_group_dev<WIN, RT>(smlo, smhi, k_group_codes(cd[o], g), 0u, pos[o], es, lutx, tables + TB_LUTC, bw, f[o], patch_rel);
#else
      decode_group_dev<WIN, RT>(smlo, smhi, k_group_codes(cd[o], g), t8[o] >> (2 * g), pos[o], es, lutx, tables + TB_LUTC, bw, f[o], patch_rel);
#endif
    }
    if (DUMP) {
#pragma unroll
      for (int o = 0; o < 2; o++)
        if (8 * o + r < nvalid) {
          u32* row = reinterpret_cast<u32*>(dump + (8 * o + r) * D);
          row[(32 * g + 2 * j) >> 1] = f[o][0]; row[(32 * g + 2 * j + 8) >> 1] = f[o][1];
          row[(32 * g + 16 + 2 * j) >> 1] = f[o][2]; row[(32 * g + 16 + 2 * j + 8) >> 1] = f[o][3];
        }
    }
    u32 qb[4];
    Q.group(g, lane, qb);
    { const u32 a[4] = {f[0][0], f[1][0], f[0][1], f[1][1]}; mma16816(sc, a, qb[0], qb[1]); }
    { const u32 a[4] = {f[0][2], f[1][2], f[0][3], f[1][3]}; mma16816(s2, a, qb[2], qb[3]); }
  }
  sc[0] += s2[0]; sc[1] += s2[1]; sc[2] += s2[2]; sc[3] += s2[3];
}

// O^T += V^T . P^T for one compressed V tile.  flrow / rowoff of V row (lane & 15) are held by lanes 16-31.
template <bool WIN, bool DUMP, bool RT = false>
__device__ __forceinline__ void v_accum(WarpAcc& A, const uint8_t* stage, const uint8_t* tables, const EscSrc<WIN>& es, u32 flrow, int rowoff,
                                        int lane, const PFrag& P, uint16_t* dump = nullptr, int nvalid = T, u32 patch_rel = 0u) {
  const int j = lane & 3, r = lane >> 2;
  const u32x2* lutx = reinterpret_cast<const u32x2*>(tables + TB_LUTX);
  u32 t4[4]; int pos[4]; uint4 sm[4]; u32 cd[6];
#pragma unroll
  for (int t = 0; t < 4; t++) {
    const int tok = 2 * j + (t & 1) + 8 * (t >> 1);
    const u32 fl = __shfl_sync(FULLM, flrow, 16 + tok);
    pos[t] = esc_part(__shfl_sync(FULLM, rowoff, 16 + tok)) + esc_prefix(fl, 4 * r) + es.off;
    t4[t] = fl >> (4 * r);
    sm[t] = *reinterpret_cast<const uint4*>(stage + ST_VSM + (lane >> 1) * SM_ROW + 64 * (lane & 1) + 16 * t);
  }
  {
    const uint2* c2 = reinterpret_cast<const uint2*>(stage + ST_VCD + 24 * lane);
    uint2 ca = c2[0], cb = c2[1], cc = c2[2];
    cd[0] = ca.x; cd[1] = ca.y; cd[2] = cb.x; cd[3] = cb.y; cd[4] = cc.x; cd[5] = cc.y;
  }
#pragma unroll
  for (int g = 0; g < 2; g++) {
    const u32x4 bw = *reinterpret_cast<const u32x4*>(tables + TB_VB + 16 * (2 * r + g));
    u32 f[4][4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const u32 smlo = g == 0 ? sm[t].x : sm[t].z, smhi = g == 0 ? sm[t].y : sm[t].w;
#if GAAC_ABLATE == 1
      f[t][0] = smlo; f[t][1] = smhi; f[t][2] = smlo ^ cd[g]; f[t][3] = smhi ^ cd[g + 3];
#elif GAAC_ABLATE == 2
      decode_group_dev<WIN, RT>(smlo, smhi, v_group_codes(cd, t, g), 0u, pos[t], es, lutx, tables + TB_LUTC, bw, f[t], patch_rel + PATCH_MAX * 8);
#else
      decode_group_dev<WIN, RT>(smlo, smhi, v_group_codes(cd, t, g), t4[t] >> (2 * g), pos[t], es, lutx, tables + TB_LUTC, bw, f[t], patch_rel + PATCH_MAX * 8);
#endif
    }
    if (DUMP) {
#pragma unroll
      for (int t = 0; t < 4; t++) {
        const int tok = 2 * j + (t & 1) + 8 * (t >> 1);
        if (tok < nvalid) {
#pragma unroll
          for (int i = 0; i < 4; i++) {                // word i = stored positions 16r + 8g + 2i, +1  <->  channels 8(8g + 2i) + r, 8(8g + 2i + 1) + r
            dump[tok * D + 8 * (8 * g + 2 * i) + r] = (uint16_t)(f[t][i] & 0xFFFFu);
            dump[tok * D + 8 * (8 * g + 2 * i + 1) + r] = (uint16_t)(f[t][i] >> 16);
          }
        }
      }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const u32 u01[4] = {f[0][2 * h], f[1][2 * h], f[2][2 * h], f[3][2 * h]};
      const u32 u23[4] = {f[0][2 * h + 1], f[1][2 * h + 1], f[2][2 * h + 1], f[3][2 * h + 1]};
      pv_words(A, 2 * g + h, u01, u23, P);
    }
  }
}

// Escape-byte offsets of the rows of a staged tile: lanes 0-15 scan the K rows, lanes 16-31 the V rows.  flrow = tag word of
// row (lane & 15) of the lane's side (0 when that side is raw), rowoff = escape bytes of the rows before it, total = rowoff
// of the row after it (lane 15 / 31 hold the tile's totals).
__device__ __forceinline__ void scan_rows(const uint8_t* stage, bool rawk, bool rawv, int lane, u32& flrow, int& rowoff, int& total) {
  const int row = lane & 15;
  const bool isv = lane >= 16;
  flrow = (isv ? rawv : rawk) ? 0u : *reinterpret_cast<const u32*>(stage + (isv ? ST_VFL : ST_KFL) + 4 * row);
  // one scan for two prefixes: escape bytes in the low half, raw groups in the high half (a tile has at most 1280 and 256 of them)
  const int sz = row_esc_bytes(flrow) + (popc(flrow & 0xAAAAAAAAu) << 16);
  int inc = sz;
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) { int v = __shfl_up_sync(FULLM, inc, d, 16); if (row >= d) inc += v; }
  rowoff = inc - sz; total = inc;
}

// Turn the raw-tier groups of a staged tile into patch-table entries, so that the group decoder needs no branch.  Lanes 0-15
// own the K rows, lanes 16-31 the V rows (as in scan_rows); a lane walks the raw groups of its row.  For each one: read the
// five payload bytes from the staged escape window, spread the 5-bit fields to byte positions, take off the 4-bit-window base
// words (the decoder adds them to every promoted group), store the two words as entry k of the side's patch table, and write k
// over the first payload byte, which is where the decoder looks for a promoted group's escape byte.  k = number of raw
// groups before this one on the tile side (rows in order, groups ascending).  side_on[0/1]: whether the K / V side takes part.
__device__ __forceinline__ void build_raw_patches(uint8_t* stage, const uint8_t* tables, uint8_t* patch, int off_k, int off_v, bool on_k, bool on_v,
                                                  u32 flrow, int rowoff, int lane) {
  const bool isv = lane >= 16;
  u32 rb = (isv ? on_v : on_k) ? (flrow & 0xAAAAAAAAu) : 0u;
  uint8_t* win = stage + ST_ZERO + (isv ? off_v : off_k);           // the tile side's first escape byte
  const uint8_t* bws = tables + (isv ? TB_VB : TB_KB);
  u32x2* ptab = reinterpret_cast<u32x2*>(patch + (isv ? PATCH_MAX * 8 : 0));
  while (__any_sync(FULLM, rb != 0u)) {
    if (rb) {
      const int bit = __ffs(rb) - 1, g = bit >> 1;                  // raw bit of group g is bit 2g + 1
      rb &= rb - 1u;
      const u32 below = flrow & ((1u << (bit - 1)) - 1u);            // tag bits of the groups before g
      const int pos = esc_part(rowoff) + popc(below & 0x55555555u) + 4 * popc(below & 0xAAAAAAAAu);
      const int k = raw_part(rowoff) + popc(below & 0xAAAAAAAAu);
      uint8_t* pl = win + pos;
      const u32 a = (u32)__cvta_generic_to_shared(pl);
      const int sh = 8 * (int)(a & 3u);
      const u32 w0 = *reinterpret_cast<const u32*>(pl - (a & 3u)), w1 = *reinterpret_cast<const u32*>(pl - (a & 3u) + 4);
      const u32 lo = funnel_r(w0, w1, sh), hi = w1 >> sh;            // bytes 0-3 and byte 4 of the payload
      const u32x4 bw = *reinterpret_cast<const u32x4*>(bws + 16 * g);
      ptab[k] = u32x2{spread_hi5_dev(lo & 0xFFFFFu) - (bw.x + bw.z), spread_hi5_dev(funnel_r(lo, hi, 20) & 0xFFFFFu) - (bw.y + bw.w)};
      *pl = (uint8_t)k;
    }
  }
  __syncwarp();
}

// Scores of a raw BF16 tile [16][128] in global memory (rows >= nvalid are not read).
template <bool DUMP>
__device__ __forceinline__ void raw_scores(float* sc, const uint16_t* kraw, int nvalid, int lane, const QFrag& Q, uint16_t* dump = nullptr) {
  const int j = lane & 3, r = lane >> 2;
  u32 qb[4];
#pragma unroll
  for (int s = 0; s < 8; s++) {
    u32 a[4];
    if ((s & 1) == 0) Q.group(s >> 1, lane, qb);
    const uint16_t* k0 = kraw + r * D + 16 * s + 2 * j;
    const uint16_t* k8 = k0 + 8 * D;
    a[0] = r < nvalid ? *reinterpret_cast<const u32*>(k0) : 0u; a[2] = r < nvalid ? *reinterpret_cast<const u32*>(k0 + 8) : 0u;
    a[1] = r + 8 < nvalid ? *reinterpret_cast<const u32*>(k8) : 0u; a[3] = r + 8 < nvalid ? *reinterpret_cast<const u32*>(k8 + 8) : 0u;
    if (DUMP) {
      if (r < nvalid) { u32* row = reinterpret_cast<u32*>(dump + r * D); row[(16 * s + 2 * j) >> 1] = a[0]; row[(16 * s + 2 * j + 8) >> 1] = a[2]; }
      if (r + 8 < nvalid) { u32* row = reinterpret_cast<u32*>(dump + (r + 8) * D); row[(16 * s + 2 * j) >> 1] = a[1]; row[(16 * s + 2 * j + 8) >> 1] = a[3]; }
    }
    mma16816(sc, a, qb[2 * (s & 1)], qb[2 * (s & 1) + 1]);
  }
}
// O^T += V^T . P^T for a raw BF16 tile.
template <bool DUMP>
__device__ __forceinline__ void raw_accum(WarpAcc& A, const uint16_t* vraw, int nvalid, int lane, const PFrag& P, uint16_t* dump = nullptr) {
  const int j = lane & 3, r = lane >> 2;
#pragma unroll
  for (int w = 0; w < 4; w++) {
    u32 u01[4], u23[4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int tok = 2 * j + (t & 1) + 8 * (t >> 1);
      const uint16_t* vr = vraw + tok * D + 8 * (4 * w) + r;
      const bool ok = tok < nvalid;
      const u32 e0 = ok ? vr[0] : 0u, e1 = ok ? vr[8] : 0u, e2 = ok ? vr[16] : 0u, e3 = ok ? vr[24] : 0u;
      u01[t] = e0 | (e1 << 16); u23[t] = e2 | (e3 << 16);
      if (DUMP && ok) {
        uint16_t* o = dump + tok * D + 8 * (4 * w) + r;
        o[0] = (uint16_t)e0; o[8] = (uint16_t)e1; o[16] = (uint16_t)e2; o[24] = (uint16_t)e3;
      }
    }
    pv_words(A, w, u01, u23, P);
  }
}

// ---- cross-GPU exchange helpers.  A receive buffer holds 8-byte entries: the low word is an fp32 value, the high word the
// number of the exchange it belongs to.  An entry is written with ONE 64-bit store and read with one 64-bit load, so a reader
// that sees the right number has the value that came with it: no flag, no fence and no second trip over NVLink is needed to
// know that a row has arrived.  Every wait is bounded: after X_WAIT_LIMIT polls (about a second) the reader gives up, so a
// missing peer never hangs the GPU.
constexpr int X_WAIT_LIMIT = 1000000;
__device__ __forceinline__ void x_store(unsigned long long* p, float v, u32 tag) {
  const unsigned long long e = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(e) : "memory");
}
__device__ __forceinline__ bool x_load(const unsigned long long* p, u32 tag, float& v) {
  for (int it = 0; it < X_WAIT_LIMIT; it++) {
    unsigned long long e;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(e) : "l"(p) : "memory");
    if ((u32)(e >> 32) == tag) { v = __uint_as_float((u32)e); return true; }
    if (it > 64) __nanosleep(100);
  }
  v = 0.f;
  return false;
}
// Wait for and merge the rows of all ranks for query head qh, element d: base = this exchange's half of the receive buffer,
// [world][rows_cap][130] entries of (m in natural-log units, l, acc[128]); same algebra as the split merge.  Returns false when
// a row did not arrive in time.
__device__ __forceinline__ bool x_merge_rows(const unsigned long long* base, int world, long rows_cap, long qh, int d, u32 tag, float& out) {
  float M = -CUDART_INF_F;
  bool ok = true;
  for (int s = 0; s < world && ok; s++) { float m; ok = x_load(base + (s * rows_cap + qh) * 130, tag, m); M = fmaxf(M, m); }   // one bound in all: stop at the first row that does not come
  float L = 0.f, Ac = 0.f;
  for (int s = 0; s < world && ok; s++) {
    const unsigned long long* pp = base + (s * rows_cap + qh) * 130;
    float ms, l, a;
    ok &= x_load(pp, tag, ms) & x_load(pp + 1, tag, l) & x_load(pp + 2 + d, tag, a);
    const float f = (ms == -CUDART_INF_F) ? 0.f : __expf(ms - M);
    L += l * f; Ac += a * f;
  }
  out = (ok && L > 0.f) ? Ac / L : 0.f;
  return ok;
}

template <bool PAGED, bool DUMP>
__global__ void __launch_bounds__(ATT_THREADS, 1) decode_attn_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int s_next, s_last;
  const int tid = threadIdx.x, lane = tid & 31, j = lane & 3, r = lane >> 2;
  const int warp = __shfl_sync(FULLM, tid >> 5, 0);   // the same value, but known to the compiler to be uniform across the warp
  const int G = p.G;
  // ---- programmatic dependent launch: the grid is launched with stream serialisation relaxed, so its CTAs can be made
  // resident while the previous kernel of the stream is still finishing (its split merge runs on a few SMs only).  Nothing
  // is read before that kernel has completed; the next kernel of the stream may be staged behind this one right away (it
  // cannot become resident before this grid's CTAs leave their SMs).  Both instructions are no-ops in a plain launch.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::);

  // Which (row, kv head, split) this CTA works on.  Normally the grid says so.  With a row order (ragged paged batches) the CTAs
  // are numbered in the order the hardware hands them out (x fastest) and that number walks the rows from the longest to the
  // shortest, all CTAs of a row together: the big CTAs start first and the small ones fill the SMs at the end.
  int bh = blockIdx.x, split = blockIdx.y, S_paged = 0;
  if (PAGED) {
    // the row's token count for the grid's own numbering; the loads of the row order travel at the same time, so a batch whose
    // order is not used pays no extra latency for having one
    S_paged = p.seq_len[bh / p.n_kv];
    if (p.row_order) {
      const int linear = blockIdx.y * gridDim.x + blockIdx.x, per_row = p.n_kv * p.nsplit;
      const int rr = linear / per_row, rem = linear - rr * per_row;
      const int2 e = p.row_order[rr], use = p.row_order[p.B];
      if (use.x) { bh = e.x * p.n_kv + rem / p.nsplit; split = rem % p.nsplit; S_paged = e.y; }
      // the numbers came out of memory: tell the compiler that they are the same in every lane (see below)
      bh = __shfl_sync(FULLM, bh, 0); split = __shfl_sync(FULLM, split, 0);
    }
  }
  const int b = bh / p.n_kv, kvh = bh % p.n_kv;

  // ---- which cache head, how many tokens, this CTA's tile range [tlo, thi)
  // (without a slot map row b reads slot b; without a length table every head holds S_uniform tokens: the two dependent
  // loads at the head of the prologue disappear for callers whose heads are all alike, which is what two Pages are)
  int S, ch = 0, TL = 0, ohk = 0, ohv = 0;
  if (PAGED) { S = S_paged; }
  else {
    const int sl = p.slot ? p.slot[b] : b;
    ch = (sl < 0 ? 0 : sl) * p.n_kv + kvh;
    const int s_ld = p.seq_len ? p.seq_len[ch] : p.S_uniform;           // these four loads do not depend on one another
    const int t_ld = p.tail_len ? p.tail_len[ch] : 0;
    ohk = p.K.head_start[ch]; ohv = p.V.head_start[ch];
    S = sl < 0 ? 0 : s_ld;
    TL = sl < 0 ? 0 : t_ld;
  }
  // These values are the same in every thread, but they were loaded from memory: passing them through a shuffle tells the
  // compiler so, and the address arithmetic built on them (one lane issues the copies) stays in uniform registers.
  S = __shfl_sync(FULLM, S, 0); ch = __shfl_sync(FULLM, ch, 0); TL = __shfl_sync(FULLM, TL, 0);
  const int ntiles = (S + 15) >> 4, chunk = (ntiles + p.nsplit - 1) / p.nsplit;
  const int tlo = min(split * chunk, ntiles), thi = min(tlo + chunk, ntiles);
  const long smh = (long)ch * p.S_pad * D, cdh = (long)ch * p.S_pad * CB, rowb = (long)ch * p.S_pad, tileb = (long)ch * (p.S_pad >> 4);
  ohk = __shfl_sync(FULLM, ohk, 0); ohv = __shfl_sync(FULLM, ohv, 0);

  // ---- addressing of this lane, and the copies of the warp's first tile: they are put in flight before the CTA builds its
  // tables so that the first tile arrives while the tables are written
  uint8_t* ring = smem + TABLE_BYTES + warp * WARP_SMEM;
  const u32 ring_s = (u32)__cvta_generic_to_shared(ring);
  LaneAddr L;
  L.ohk = ohk; L.ohv = ohv;
  L.availk = PAGED ? 0 : (int)min((long)(1 << 30), p.K.ovf_bytes - ohk); L.availv = PAGED ? 0 : (int)min((long)(1 << 30), p.V.ovf_bytes - ohv);
  const int* metak = reinterpret_cast<const int*>(smem + TB_META);
  const int* metav = metak + META_TILES;
  auto global_meta = [&](int tile) -> TileMeta {
    if (PAGED) { const int pc = p.bt[(long)b * p.bt_stride + tile] * (2 * p.n_kv) + 2 * kvh; return TileMeta{p.mt[pc], p.mt[pc + 1]}; }
    return TileMeta{p.K.tile_off[tileb + tile], p.V.tile_off[tileb + tile]};
  };
  auto meta_of = [&](int tile) -> TileMeta {          // valid after the CTA has staged its metadata
    if (tile - tlo < META_TILES) return TileMeta{metak[tile - tlo], metav[tile - tlo]};
    return global_meta(tile);
  };
  // Slot layout, escape window of a tile whose escapes start `m` bytes into the head's escape bytes, in 32-bit arithmetic:
  // w16 = its first byte's offset inside a 16-byte unit, n = bytes of the copy from the unit's start (a multiple of 16, at most
  // ESC_COPY, inside the allocation; 0 when the unit starts before the allocation).
  const int a16k = PAGED ? 0 : (int)((reinterpret_cast<uintptr_t>(p.K.ovf) + (unsigned)ohk) & 15), a16v = PAGED ? 0 : (int)((reinterpret_cast<uintptr_t>(p.V.ovf) + (unsigned)ohv) & 15);
  auto esc_win = [&](bool vside, int m, int& w16, int& n) {
    w16 = ((vside ? a16v : a16k) + m) & 15;
    const int to_end = (vside ? L.availv : L.availk) - m + w16;                 // bytes from the unit's start to the end of the allocation
    n = ((vside ? L.ohv : L.ohk) + m < w16) ? 0 : max(0, min(ESC_COPY, to_end & ~15));
  };
  auto bulk_issue = [&](u32 st, int tile, const TileMeta& m) {                  // executed by lane 0
    const u32 mb = st + ST_MBAR;
    // the stage may have been written through ordinary stores (patch numbers in its escape window): order those before the
    // copy engine's writes to the same bytes
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (PAGED) {
      const u32 n = (u32)min(p.TS, SLOT_OVF_OFF + ESC_COPY);                    // a slot is one contiguous piece, escapes included
      mbar_expect_tx(mb, (m.mk >= 0 ? n : 0u) + (m.mv >= 0 ? n : 0u));
      if (m.mk >= 0) bulk_g2s(st + ST_KSM, p.buf + (long)m.mk * p.TS, n, mb);
      if (m.mv >= 0) bulk_g2s(st + ST_VSM, p.buf + (long)m.mv * p.TS, n, mb);
    } else {
      int wk, nk, wv, nv;
      esc_win(false, m.mk, wk, nk); esc_win(true, m.mv, wv, nv);
      mbar_expect_tx(mb, (u32)(2 * (TILE_SM + TILE_CD + 4 * T) + nk + nv));
      const long so = smh + (long)tile * TILE_SM, co = cdh + (long)tile * TILE_CD, fo = (rowb + (long)tile * T) * 4;
      bulk_g2s(st + ST_KSM, p.K.sm + so, TILE_SM, mb); bulk_g2s(st + ST_VSM, p.V.sm + so, TILE_SM, mb);
      bulk_g2s(st + ST_KCD, p.K.codes + co, TILE_CD, mb); bulk_g2s(st + ST_VCD, p.V.codes + co, TILE_CD, mb);
      bulk_g2s(st + ST_KFL, reinterpret_cast<const uint8_t*>(p.K.flags) + fo, 4 * T, mb);
      bulk_g2s(st + ST_VFL, reinterpret_cast<const uint8_t*>(p.V.flags) + fo, 4 * T, mb);
      if (nk > 0) bulk_g2s(st + ST_KESC, p.K.ovf + ((long)L.ohk + m.mk - wk), (u32)nk, mb);
      if (nv > 0) bulk_g2s(st + ST_VESC, p.V.ovf + ((long)L.ohv + m.mv - wv), (u32)nv, mb);
    }
  };
  // Escape bytes of a staged side as the group decoder reads them: first escape byte in global memory, offset from the stage's
  // zero byte to the first escape byte, staged bytes counted from the first escape byte
  auto staged_escapes = [&](bool vside, int m, int& off, int& avail) {
    const int base = (vside ? ST_VESC : ST_KESC) - ST_ZERO;
    if (PAGED) { off = base; avail = min(p.ovf_slot, min(p.TS, SLOT_OVF_OFF + ESC_COPY) - SLOT_OVF_OFF); }
    else { int w16, n; esc_win(vside, m, w16, n); off = base + w16; avail = n - w16; }
  };
  auto global_escapes = [&](bool vside, int m) -> const uint8_t* {            // only tiles whose escapes exceed the window get here
    if (PAGED) return p.buf + (long)m * p.TS + SLOT_OVF_OFF;
    return (vside ? p.V.ovf : p.K.ovf) + ((long)(vside ? L.ohv : L.ohk) + m);
  };
  // ---- prologue.  Everything that reads global memory is put in flight first and consumed afterwards: the payload of the
  // warp's first tile (needs no metadata in the slot layout), the tile's metadata, the metadata of the CTA's range, the
  // query rows; then the tables are built while those loads travel.
  int tile = tlo + warp;
  TileMeta cur{0, 0};
  if (lane == 0) {                                    // one barrier per stage, one arrival (this lane's) per phase; 8 zero bytes beside it
    mbar_init(ring_s + ST_MBAR, 1); mbar_init(ring_s + STAGE_BYTES + ST_MBAR, 1);
    *reinterpret_cast<unsigned long long*>(ring + ST_ZERO) = 0ull; *reinterpret_cast<unsigned long long*>(ring + STAGE_BYTES + ST_ZERO) = 0ull;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  if (tile < thi) {
    if (PAGED) { cur = global_meta(tile); if (lane == 0) bulk_issue(ring_s, tile, cur); }
    else {
      // slot layout: the six payload copies need no metadata and leave at once; the escape windows (and the barrier's arrival)
      // follow further down, when the tile's escape offsets have come back from global memory
      if (lane == 0) {
        const u32 mb = ring_s + ST_MBAR;
        const long so = smh + (long)tile * TILE_SM, co = cdh + (long)tile * TILE_CD, fo = (rowb + (long)tile * T) * 4;
        mbar_add_tx(mb, 2 * (TILE_SM + TILE_CD + 4 * T));
        bulk_g2s(ring_s + ST_KSM, p.K.sm + so, TILE_SM, mb); bulk_g2s(ring_s + ST_VSM, p.V.sm + so, TILE_SM, mb);
        bulk_g2s(ring_s + ST_KCD, p.K.codes + co, TILE_CD, mb); bulk_g2s(ring_s + ST_VCD, p.V.codes + co, TILE_CD, mb);
        bulk_g2s(ring_s + ST_KFL, reinterpret_cast<const uint8_t*>(p.K.flags) + fo, 4 * T, mb);
        bulk_g2s(ring_s + ST_VFL, reinterpret_cast<const uint8_t*>(p.V.flags) + fo, 4 * T, mb);
      }
      cur = global_meta(tile);
    }
  }
  int* mk_s = reinterpret_cast<int*>(smem + TB_META);
  int* mv_s = mk_s + META_TILES;
  const int nstaged = min(thi - tlo, META_TILES);
  TileMeta m_first{0, 0};
  if (tid < nstaged) m_first = global_meta(tlo + tid);
  QFrag Q;
#if GAAC_QSMEM
  Q.tab = reinterpret_cast<const uint4*>(smem + TB_Q);
  uint4 q_mine = make_uint4(0u, 0u, 0u, 0u);            // threads 0..127 load one table entry each: K group tid >> 5 of lane tid & 31
  if (tid < 128) {
    const int gg = tid >> 5, jj = tid & 3, rr = (tid & 31) >> 2;
    if (rr < G) {
      const uint16_t* qp = p.q + ((long)b * p.n_q + kvh * G + rr) * D + 32 * gg + 2 * jj;
      q_mine = make_uint4(*reinterpret_cast<const u32*>(qp), *reinterpret_cast<const u32*>(qp + 8), *reinterpret_cast<const u32*>(qp + 16), *reinterpret_cast<const u32*>(qp + 24));
    }
  }
#else
  {
    const bool ok = r < G;
    const uint16_t* qp = p.q + ((long)b * p.n_q + kvh * G + (ok ? r : 0)) * D;
#pragma unroll
    for (int s = 0; s < 8; s++) {
      Q.qa[s][0] = ok ? *reinterpret_cast<const u32*>(qp + 16 * s + 2 * j) : 0u;
      Q.qa[s][1] = ok ? *reinterpret_cast<const u32*>(qp + 16 * s + 2 * j + 8) : 0u;
    }
  }
#endif
  // ---- CTA tables: escape-byte table, code table, per-lane-class base words {b3lo, b3hi, b4lo-b3lo, b4hi-b3hi} per group,
  // zero pads, per-tile metadata of the range (escape offsets or mode-table entries, so that the main loop never waits on a
  // dependent global load)
  {
    const int brow = PAGED ? kvh : ch % p.n_base_rows;
    const uint8_t* b3k = (PAGED ? p.b3k : p.K.base3) + brow * D; const uint8_t* b4k = (PAGED ? p.b4k : p.K.base4) + brow * D;
    const uint8_t* b3v = (PAGED ? p.b3v : p.V.base3) + brow * D; const uint8_t* b4v = (PAGED ? p.b4v : p.V.base4) + brow * D;
    constexpr int KB_T0 = ATT_THREADS >= 320 ? 256 : 0, VB_T0 = KB_T0 + 32;       // which threads build the base words (beside the escape-byte table when the CTA is small)
    if (tid >= KB_T0 && tid < KB_T0 + 16) {           // K: lane class jj, group gg -> words 2gg, 2gg+1
      const int t = tid - KB_T0, jj = t >> 2, gg = t & 3; u32 w3[8], w4[8];
      k_base_words(b3k, jj, w3); k_base_words(b4k, jj, w4);
      *reinterpret_cast<u32x4*>(smem + TB_KB + 16 * t) = u32x4{w3[2 * gg], w3[2 * gg + 1], w4[2 * gg] - w3[2 * gg], w4[2 * gg + 1] - w3[2 * gg + 1]};
    } else if (tid >= VB_T0 && tid < VB_T0 + 16) {    // V: lane class rr, group gg
      const int t = tid - VB_T0, rr = t >> 1, gg = t & 1; u32 w3[4], w4[4];
      v_base_words(b3v, rr, w3); v_base_words(b4v, rr, w4);
      *reinterpret_cast<u32x4*>(smem + TB_VB + 16 * t) = u32x4{w3[2 * gg], w3[2 * gg + 1], w4[2 * gg] - w3[2 * gg], w4[2 * gg + 1] - w3[2 * gg + 1]};
    }
    if (tid < 256) fill_lutx(reinterpret_cast<u32x2*>(smem + TB_LUTX), tid);
#if GAAC_QSMEM
    if (tid < 128) reinterpret_cast<uint4*>(smem + TB_Q)[tid] = q_mine;
#endif
#if GAAC_LUTC
    for (int i = tid; i < 4096; i += ATT_THREADS) reinterpret_cast<u32*>(smem + TB_LUTC)[i] = spread_codes4((u32)i);
#endif
    if (tid == 0) s_next = tlo + ATT_WARPS;           // tiles tlo .. tlo+W-1 go to warps 0..W-1, the rest is handed out on demand
    if (tid < nstaged) { mk_s[tid] = m_first.mk; mv_s[tid] = m_first.mv; }
    for (int i = tid + ATT_THREADS; i < nstaged; i += ATT_THREADS) { const TileMeta m = global_meta(tlo + i); mk_s[i] = m.mk; mv_s[i] = m.mv; }
  }
  if (!PAGED && tile < thi && lane == 0) {
    const u32 mb = ring_s + ST_MBAR;
    int wk, nk, wv, nv;
    esc_win(false, cur.mk, wk, nk); esc_win(true, cur.mv, wv, nv);
    if (nk + nv > 0) mbar_add_tx(mb, (u32)(nk + nv));
    if (nk > 0) bulk_g2s(ring_s + ST_KESC, p.K.ovf + ((long)L.ohk + cur.mk - wk), (u32)nk, mb);
    if (nv > 0) bulk_g2s(ring_s + ST_VESC, p.V.ovf + ((long)L.ohv + cur.mv - wv), (u32)nv, mb);
    mbar_arrive(mb);
  }
  WarpAcc A;
#pragma unroll
  for (int n = 0; n < 8; n++) A.acc[n][0] = A.acc[n][1] = A.acc[n][2] = A.acc[n][3] = 0.f;
  A.m0 = A.m1 = -CUDART_INF_F; A.l0 = A.l1 = 0.f;
  __syncthreads();

  uint16_t* const dump_k = DUMP ? p.dump_k + (long)bh * p.dump_S * D : nullptr;
  uint16_t* const dump_v = DUMP ? p.dump_v + (long)bh * p.dump_S * D : nullptr;
  // ---- main loop.  The warp's first tile is tlo + warp; every further tile is taken from the CTA's counter while the
  // current one is being consumed, one tile ahead of its use, so fast and slow warps finish within about one tile of each
  // other.  The counter is read at the top of the iteration and its value used after the K half, which hides the latency
  // of the shared-memory atomic; the copies of the next tile are issued between the K half and the V half.
  int stg = 0;
  u32 phase = 0;                                       // bit s: parity of the phase of stage s that is waited for next
#if GAAC_DEEP
  // the warp's second tile goes into the other stage right away; from then on the stage a tile leaves is refilled, as soon as the
  // tile is done, with the tile after the next one, so the copies of a tile have a whole tile's time to arrive
  int tile_b = thi; TileMeta meta_b{0, 0};
  if (tile < thi) {
    int t = 0;
    if (lane == 0) t = atomicAdd(&s_next, 1);
    tile_b = __shfl_sync(FULLM, t, 0);
    if (tile_b < thi) { meta_b = meta_of(tile_b); if (lane == 0) bulk_issue(ring_s + STAGE_BYTES, tile_b, meta_b); }
  }
#endif
  while (tile < thi) {
    int t1 = 0;
    if (lane == 0) t1 = atomicAdd(&s_next, 1);
    if (!__all_sync(FULLM, mbar_wait(ring_s + stg * STAGE_BYTES + ST_MBAR, (phase >> stg) & 1u))) {     // the whole warp gives up together
      if (lane == 0) atomicExch(p.err, 1);
      break;
    }
    phase ^= 1u << stg;
    const uint8_t* stage = ring + stg * STAGE_BYTES;
    const int nvalid = min(T, S - tile * T);
    const bool rawk = PAGED && cur.mk < 0, rawv = PAGED && cur.mv < 0;
    u32 flrow; int rowoff, total;
    scan_rows(stage, rawk, rawv, lane, flrow, rowoff, total);
    // which decoder each side takes: the staged window (branch-free, raw groups through the patch table) when the side's escape
    // bytes all fit the window and it has at most PATCH_MAX raw groups; else the one that reads escapes from global memory
    int off_k = 0, off_v = 0, avail_k = 0, avail_v = 0;
    if (!rawk) staged_escapes(false, cur.mk, off_k, avail_k);
    if (!rawv) staged_escapes(true, cur.mv, off_v, avail_v);
    const int tot_k = __shfl_sync(FULLM, total, 15), tot_v = __shfl_sync(FULLM, total, 31);
    const bool win_k = !rawk && esc_part(tot_k) + 8 <= avail_k && (!GAAC_RAWPATCH || raw_part(tot_k) <= PATCH_MAX);     // +8: a raw payload is read as two aligned words
    const bool win_v = !rawv && esc_part(tot_v) + 8 <= avail_v && (!GAAC_RAWPATCH || raw_part(tot_v) <= PATCH_MAX);
    uint8_t* const patch = ring + NSTAGE * STAGE_BYTES;
    const u32 patch_rel = (u32)(patch - (smem + TB_LUTX));
#if GAAC_RAWPATCH
    if ((win_k && raw_part(tot_k) > 0) || (win_v && raw_part(tot_v) > 0))
      build_raw_patches(ring + stg * STAGE_BYTES, smem, patch, off_k, off_v, win_k, win_v, flrow, rowoff, lane);
#endif
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    if (!rawk) {
      if (win_k)
        k_scores<true, DUMP, GAAC_RAWPATCH != 0>(sc, stage, smem, EscSrc<true>{stage + ST_ZERO, nullptr, off_k}, flrow, rowoff, lane, Q, dump_k + (long)tile * T * D, nvalid, patch_rel);
      else
        k_scores<false, DUMP>(sc, stage, smem, EscSrc<false>{nullptr, global_escapes(false, cur.mk), 0}, flrow, rowoff, lane, Q, dump_k + (long)tile * T * D, nvalid);
    } else {
      raw_scores<DUMP>(sc, p.raw + (long)(~cur.mk) * (T * D), nvalid, lane, Q, dump_k + (long)tile * T * D);
    }
    t1 = __shfl_sync(FULLM, t1, 0);
    TileMeta nxt{0, 0};
#if !GAAC_DEEP
    if (t1 < thi) {
      nxt = meta_of(t1);
      const u32 st = ring_s + (stg ^ 1) * STAGE_BYTES;
      if (lane == 0) bulk_issue(st, t1, nxt);
    }
#endif
    PFrag P;
    if (nvalid == T) softmax_step<true>(A, sc, p.scale_log2, nvalid, lane, P);
    else softmax_step<false>(A, sc, p.scale_log2, nvalid, lane, P);
    if (!rawv) {
      if (win_v)
        v_accum<true, DUMP, GAAC_RAWPATCH != 0>(A, stage, smem, EscSrc<true>{stage + ST_ZERO, nullptr, off_v}, flrow, rowoff, lane, P, dump_v + (long)tile * T * D, nvalid, patch_rel);
      else
        v_accum<false, DUMP>(A, stage, smem, EscSrc<false>{nullptr, global_escapes(true, cur.mv), 0}, flrow, rowoff, lane, P, dump_v + (long)tile * T * D, nvalid);
    } else {
      raw_accum<DUMP>(A, p.raw + (long)(~cur.mv) * (T * D), nvalid, lane, P, dump_v + (long)tile * T * D);
    }
#if GAAC_DEEP
    __syncwarp();                                      // every lane has read what it needs of this stage
    if (t1 < thi) { nxt = meta_of(t1); if (lane == 0) bulk_issue(ring_s + stg * STAGE_BYTES, t1, nxt); }
    cur = meta_b; tile = tile_b; meta_b = nxt; tile_b = t1; stg ^= 1;
#else
    cur = nxt; stg ^= 1; tile = t1;
#endif
  }
  // ---- slot layout: the raw BF16 tail belongs to the last split's warp 0
  if (!PAGED && TL > 0 && split == p.nsplit - 1 && warp == 0) {
    const uint16_t* kraw = reinterpret_cast<const uint16_t*>(p.K.tail) + (long)ch * p.tail_cap * D;
    const uint16_t* vraw = reinterpret_cast<const uint16_t*>(p.V.tail) + (long)ch * p.tail_cap * D;
    for (int t0 = 0; t0 < TL; t0 += T) {
      const int nvalid = min(T, TL - t0);
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
      raw_scores<DUMP>(sc, kraw, nvalid, lane, Q, dump_k + ((long)S + t0) * D);
      PFrag P;
      softmax_step<false>(A, sc, p.scale_log2, nvalid, lane, P);
      raw_accum<DUMP>(A, vraw, nvalid, lane, P, dump_v + ((long)S + t0) * D);
      kraw += T * D; vraw += T * D;
    }
  }

  // ---- merge the warps of the CTA (the rings are free now)
  __syncthreads();
  constexpr int ACC_LD = D + 4;                                  // row stride of the staged accumulators: 4j + r banks, conflict-free stores
  float* sh_m = reinterpret_cast<float*>(smem + TABLE_BYTES);    // [W][8]
  float* sh_l = sh_m + ATT_WARPS * 8;                            // [W][8]
  float* sh_acc = sh_l + ATT_WARPS * 8;                          // [W][8][ACC_LD]
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) { A.l0 += __shfl_xor_sync(FULLM, A.l0, o); A.l1 += __shfl_xor_sync(FULLM, A.l1, o); }
  if (r == 0) { sh_m[warp * 8 + 2 * j] = A.m0; sh_l[warp * 8 + 2 * j] = A.l0; sh_m[warp * 8 + 2 * j + 1] = A.m1; sh_l[warp * 8 + 2 * j + 1] = A.l1; }
  if (2 * j < G) {                                               // heads 2j, 2j+1 (the second may be a padding head: stored, never read)
#pragma unroll
    for (int n = 0; n < 8; n++) {
      float* a0 = sh_acc + ((warp * 8 + 2 * j) * ACC_LD) + 16 * n + r;
      a0[0] = A.acc[n][0]; a0[ACC_LD] = A.acc[n][1]; a0[8] = A.acc[n][2]; a0[ACC_LD + 8] = A.acc[n][3];
    }
  }
  __syncthreads();
  const int NS = p.nsplit;
  {
    const int d = tid & 127;
    for (int g = tid >> 7; g < G; g += ATT_THREADS / 128) {
      float M = -CUDART_INF_F;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; w++) M = fmaxf(M, sh_m[w * 8 + g]);
      float Lc = 0.f, Ac = 0.f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; w++) {
        const float mw = sh_m[w * 8 + g];
        const float f = (mw == -CUDART_INF_F) ? 0.f : fast_exp2(mw - M);
        Lc += sh_l[w * 8 + g] * f; Ac += sh_acc[(w * 8 + g) * ACC_LD + d] * f;
      }
      const long qh = (long)b * p.n_q + kvh * G + g, pidx = qh * NS + split;
      if (d == 0) { p.pm[pidx] = M; p.pl[pidx] = Lc; }
      p.pa[pidx * D + d] = Ac;
    }
  }
  // ---- the last CTA of this (row, kv head) merges the splits.  The ticket is taken with an acquire-release atomic at GPU scope
  // by one thread between two CTA barriers: the barrier before it orders every thread's partial stores before the release, the
  // barrier after it orders the acquire before every thread's loads of the other CTAs' partials - no per-thread fence is needed.
  __syncthreads();
  if (tid == 0) {
    int ticket;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + bh) : "memory");
    s_last = (ticket == NS - 1);
    if (s_last) p.counters[bh] = 0;                 // leave the counter ready for the next call
  }
  __syncthreads();
  if (!s_last) return;
  // All loads below are independent of one another (no per-split dependent chain): scale factors first, then the weighted sum
  // with one warp per split and 16-byte loads, then a cross-warp sum in shared memory.
  {
    float* c_f = reinterpret_cast<float*>(smem + TABLE_BYTES);           // [G][NS]  m, then exp2(m - M)
    float* c_l = c_f + 8 * NS;                                            // [G][NS]  l
    float* c_ML = c_l + 8 * NS;                                           // [8][2]   M, L per head
    float* c_red = c_ML + 16;                                             // [W][G][128] (NS <= 1024 keeps this inside the ring area)
    const long qh0 = (long)b * p.n_q + kvh * G;
    for (int i = tid; i < G * NS; i += ATT_THREADS) { c_f[i] = __ldcg(p.pm + qh0 * NS + i); c_l[i] = __ldcg(p.pl + qh0 * NS + i); }
    float4 pre[8];                                                        // split `warp` of every head, in flight while M and L are computed
#pragma unroll
    for (int g = 0; g < 8; g++)
      pre[g] = (g < G && warp < NS) ? __ldcg(reinterpret_cast<const float4*>(p.pa + ((qh0 + g) * NS + warp) * D) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();
    if (warp < G) {
      float M = -CUDART_INF_F;
      for (int s2 = lane; s2 < NS; s2 += 32) M = fmaxf(M, c_f[warp * NS + s2]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(FULLM, M, o));
      float L = 0.f;
      for (int s2 = lane; s2 < NS; s2 += 32) {
        const float ms = c_f[warp * NS + s2];
        const float f = (ms == -CUDART_INF_F) ? 0.f : fast_exp2(ms - M);
        c_f[warp * NS + s2] = f; L += c_l[warp * NS + s2] * f;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(FULLM, L, o);
      if (lane == 0) { c_ML[2 * warp] = M; c_ML[2 * warp + 1] = L; }
    }
    __syncthreads();
    float4 acc4[8];
#pragma unroll
    for (int g = 0; g < 8; g++) {
      const float f = (g < G && warp < NS) ? c_f[g * NS + warp] : 0.f;
      acc4[g] = make_float4(pre[g].x * f, pre[g].y * f, pre[g].z * f, pre[g].w * f);
    }
    for (int s2 = warp + ATT_WARPS; s2 < NS; s2 += ATT_WARPS) {
#pragma unroll
      for (int g = 0; g < 8; g++) {
        if (g < G) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(p.pa + ((qh0 + g) * NS + s2) * D) + lane);
          const float f = c_f[g * NS + s2];
          acc4[g].x += v.x * f; acc4[g].y += v.y * f; acc4[g].z += v.z * f; acc4[g].w += v.w * f;
        }
      }
    }
#pragma unroll
    for (int g = 0; g < 8; g++)
      if (g < G) *reinterpret_cast<float4*>(c_red + ((warp * 8 + g) * D) + 4 * lane) = acc4[g];
    __syncthreads();
    const int d = tid & 127;
    const int x_ep = p.x_recv ? __ldcg(p.x_epoch) : 0;         // number of this exchange - 1; advanced only after every group has read it
    for (int g = tid >> 7; g < G; g += ATT_THREADS / 128) {
      float Ac = 0.f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; w++) Ac += c_red[(w * 8 + g) * D + d];
      const float M = c_ML[2 * g], L = c_ML[2 * g + 1];
      const long qh = qh0 + g;
      if (p.x_recv) {                                // the same partial, pushed to every rank's receive buffer over NVLink
        const long row = ((long)((x_ep & 1) * p.x_world + p.x_rank) * p.x_rows_cap + qh) * 130;
        for (int rk = 0; rk < p.x_world; rk++) {
          unsigned long long* o = p.x_recv[rk] + row;
          if (d == 0) { x_store(o, M * LN2, (u32)x_ep + 1u); x_store(o + 1, L, (u32)x_ep + 1u); }
          x_store(o + 2 + d, Ac, (u32)x_ep + 1u);
        }
      } else if (p.part) {                           // un-normalised partial for a cross-GPU merge: m in natural-log units
        float* o = p.part + qh * 130;
        if (d == 0) { o[0] = M * LN2; o[1] = L; }
        o[2 + d] = Ac;
      } else {
        const float v = L > 0.f ? Ac / L : 0.f;
        p.out[qh * D + d] = __bfloat16_as_ushort(__float2bfloat16(v));
        if (p.out_f32) p.out_f32[qh * D + d] = v;
      }
    }
    if (p.x_recv) {
      // Every entry carries the exchange number, so nothing else announces the rows (see x_store / x_load).
      if (!p.x_fused) return;                        // the wait-and-merge runs as its own launch (gaac_exchange_merge)
      // ---- fused: wait (bounded) for the rows of this group from every rank, merge them, write the output
      const unsigned long long* base = p.x_recv[p.x_rank] + (long)(x_ep & 1) * p.x_world * p.x_rows_cap * 130;
      float v[2] = {0.f, 0.f};
      int bad = 0;
      for (int g = tid >> 7, i = 0; g < G; g += ATT_THREADS / 128, i++)
        bad |= !x_merge_rows(base, p.x_world, p.x_rows_cap, qh0 + g, d, (u32)x_ep + 1u, v[i]);
      const int any_bad = __syncthreads_or(bad);     // a group whose rows did not all arrive is reported and comes back as zeros
      if (any_bad && tid == 0) atomicExch(p.x_err, 1);
      for (int g = tid >> 7, i = 0; g < G; g += ATT_THREADS / 128, i++) {
        const long qh = qh0 + g;
        const float o = any_bad ? 0.f : v[i];
        if (p.out) p.out[qh * D + d] = __bfloat16_as_ushort(__float2bfloat16(o));
        if (p.out_f32) p.out_f32[qh * D + d] = o;
      }
      // the exchange number advances when every group of this launch is through (each has read it by then)
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        if (atomicAdd(p.x_ticket, 1) == (int)gridDim.x - 1) { *p.x_ticket = 0; __threadfence(); atomicAdd(p.x_epoch, 1); }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ head_dim 256, paged layout
// A 256-dim head is stored as two 128-dim half-heads in neighbouring tile slots, each with its own bases
// (gaac/vllm/paged_kernel256.py:1-4): block = 2*n_kv half-heads x {K, V}, half-head hh = 2*kvh + half.  Two warps form a pair that
// streams the same tiles: each warp owns one half - it stages and rebuilds its half's K tile, which yields a partial score, and
// its half's V tile, which yields its 128 output dimensions.  The two partial scores meet in shared memory once per tile (one
// 64-thread named barrier; the exchange slots alternate with the tile's parity so one barrier per tile is enough), after which
// both warps run the same softmax step on the same numbers.  Tiles are handed to PAIRS from the CTA's counter; the even warp
// takes the number and passes it through the exchange slot.  A warp whose bounded wait on its copies runs out says so in
// the same slot, so that both warps of the pair leave the loop together and nobody is left at the barrier.
// Output: un-normalised partials of "virtual heads" vq = 2 * query head + half, i.e. exactly the layout gaac_combine turns into
// out [B, n_q, 256].
static_assert(GAAC_LUTC == 0 && ATT_WARPS % 2 == 0, "the 256-dim kernel uses the arithmetic code spreading and warp pairs");
constexpr int T256_HALF = 2048 + 256 + 256;                       // per half: escape-byte table, K base words, V base words (same offsets as the CTA tables above)
constexpr int XCH_PAR_BYTES = 2 * 32 * 16 + 16;                    // one parity: two halves x 32 lanes x float4, then {next tile, fail flag of half 0, of half 1, -}
constexpr int T256_XCH = 2 * T256_HALF;
constexpr int TABLE256_BYTES = T256_XCH + (ATT_WARPS / 2) * 2 * XCH_PAR_BYTES;
constexpr int ATT256_SMEM = TABLE256_BYTES + ATT_WARPS * WARP_SMEM;
static_assert(TB_KB == 2048 && TB_VB == 2048 + 256 && TABLE256_BYTES % 16 == 0 && ATT256_SMEM + 64 <= 232448, "table layout shared with the 128-dim kernel; one CTA per SM");

__global__ void __launch_bounds__(ATT_THREADS, 1) paged256_attn_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int s_next;
  const int bh = blockIdx.x, split = blockIdx.y, tid = threadIdx.x, lane = tid & 31, j = lane & 3, r = lane >> 2;
  const int warp = __shfl_sync(FULLM, tid >> 5, 0);
  const int hf = warp & 1, pair = warp >> 1;
  const int b = bh / p.n_kv, kvh = bh % p.n_kv, G = p.G, hh = 2 * kvh + hf, NT = 4 * p.n_kv;    // p.n_kv = 256-dim kv heads; NT tile slots per block
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::);
  const int S = __shfl_sync(FULLM, p.seq_len[b], 0);
  const int ntiles = (S + 15) >> 4, chunk = (ntiles + p.nsplit - 1) / p.nsplit;
  const int tlo = min(split * chunk, ntiles), thi = min(tlo + chunk, ntiles);
  uint8_t* ring = smem + TABLE256_BYTES + warp * WARP_SMEM;
  const u32 ring_s = (u32)__cvta_generic_to_shared(ring);
  const uint8_t* tables = smem + hf * T256_HALF;
  uint8_t* xch = smem + T256_XCH + pair * (2 * XCH_PAR_BYTES);
  auto meta = [&](int tile) -> TileMeta { const int pc = p.bt[(long)b * p.bt_stride + tile] * NT + 2 * hh; return TileMeta{p.mt[pc], p.mt[pc + 1]}; };
  auto issue = [&](u32 st, const TileMeta& m) {                                // executed by lane 0
    const u32 mb = st + ST_MBAR, n = (u32)min(p.TS, SLOT_OVF_OFF + ESC_COPY);
    mbar_expect_tx(mb, (m.mk >= 0 ? n : 0u) + (m.mv >= 0 ? n : 0u));
    if (m.mk >= 0) bulk_g2s(st + ST_KSM, p.buf + (long)m.mk * p.TS, n, mb);
    if (m.mv >= 0) bulk_g2s(st + ST_VSM, p.buf + (long)m.mv * p.TS, n, mb);
  };
  if (lane == 0) {
    mbar_init(ring_s + ST_MBAR, 1); mbar_init(ring_s + STAGE_BYTES + ST_MBAR, 1);
    *reinterpret_cast<unsigned long long*>(ring + ST_ZERO) = 0ull; *reinterpret_cast<unsigned long long*>(ring + STAGE_BYTES + ST_ZERO) = 0ull;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  int tile = tlo + pair;
  TileMeta cur{0, 0};
  if (tile < thi) { cur = meta(tile); if (lane == 0) issue(ring_s, cur); }
  QFrag Q;
#if GAAC_QSMEM
#error "the 256-dim kernel keeps the query fragments in registers"
#else
  {
    const bool ok = r < G;
    const uint16_t* qp = p.q + ((long)b * p.n_q + kvh * G + (ok ? r : 0)) * (2 * D) + hf * D;
#pragma unroll
    for (int s = 0; s < 8; s++) {
      Q.qa[s][0] = ok ? *reinterpret_cast<const u32*>(qp + 16 * s + 2 * j) : 0u;
      Q.qa[s][1] = ok ? *reinterpret_cast<const u32*>(qp + 16 * s + 2 * j + 8) : 0u;
    }
  }
#endif
  {   // tables of both halves; exchange slots start out zero
    if (tid < 256) { fill_lutx(reinterpret_cast<u32x2*>(smem + TB_LUTX), tid); fill_lutx(reinterpret_cast<u32x2*>(smem + T256_HALF + TB_LUTX), tid); }
    constexpr int KB_T0 = ATT_THREADS >= 320 ? 256 : 0, VB_T0 = KB_T0 + 32;
    if (tid >= KB_T0 && tid < KB_T0 + 32) {           // K: half, lane class jj, group gg
      const int t = tid - KB_T0, h2 = t >> 4, jj = (t >> 2) & 3, gg = t & 3; u32 w3[8], w4[8];
      const int row = 2 * kvh + h2;
      k_base_words(p.b3k + row * D, jj, w3); k_base_words(p.b4k + row * D, jj, w4);
      *reinterpret_cast<u32x4*>(smem + h2 * T256_HALF + TB_KB + 16 * (t & 15)) = u32x4{w3[2 * gg], w3[2 * gg + 1], w4[2 * gg] - w3[2 * gg], w4[2 * gg + 1] - w3[2 * gg + 1]};
    } else if (tid >= VB_T0 && tid < VB_T0 + 32) {    // V: half, lane class rr, group gg
      const int t = tid - VB_T0, h2 = t >> 4, rr = (t >> 1) & 7, gg = t & 1; u32 w3[4], w4[4];
      const int row = 2 * kvh + h2;
      v_base_words(p.b3v + row * D, rr, w3); v_base_words(p.b4v + row * D, rr, w4);
      *reinterpret_cast<u32x4*>(smem + h2 * T256_HALF + TB_VB + 16 * (t & 15)) = u32x4{w3[2 * gg], w3[2 * gg + 1], w4[2 * gg] - w3[2 * gg], w4[2 * gg + 1] - w3[2 * gg + 1]};
    }
    for (int i = tid; i < (ATT_WARPS / 2) * 2 * XCH_PAR_BYTES / 4; i += ATT_THREADS) reinterpret_cast<u32*>(smem + T256_XCH)[i] = 0u;
    if (tid == 0) s_next = tlo + ATT_WARPS / 2;       // tiles tlo .. tlo + pairs - 1 go to the pairs in order, the rest is handed out on demand
  }
  WarpAcc A;
#pragma unroll
  for (int n = 0; n < 8; n++) A.acc[n][0] = A.acc[n][1] = A.acc[n][2] = A.acc[n][3] = 0.f;
  A.m0 = A.m1 = -CUDART_INF_F; A.l0 = A.l1 = 0.f;
  __syncthreads();

  int stg = 0, par = 0;
  u32 phase = 0;
  const int esc_off = ST_KESC - ST_ZERO, esc_off_v = ST_VESC - ST_ZERO;
  const int esc_avail = min(p.ovf_slot, min(p.TS, SLOT_OVF_OFF + ESC_COPY) - SLOT_OVF_OFF);
  while (tile < thi) {
    int t1 = 0;
    if (hf == 0 && lane == 0) t1 = atomicAdd(&s_next, 1);
    const bool ok = __all_sync(FULLM, mbar_wait(ring_s + stg * STAGE_BYTES + ST_MBAR, (phase >> stg) & 1u));
    phase ^= 1u << stg;
    const uint8_t* stage = ring + stg * STAGE_BYTES;
    const int nvalid = min(T, S - tile * T);
    const bool rawk = cur.mk < 0, rawv = cur.mv < 0;
    u32 flrow = 0; int rowoff = 0, total = 0;
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok) {
      scan_rows(stage, rawk, rawv, lane, flrow, rowoff, total);
      if (!rawk) {
        if (esc_part(__shfl_sync(FULLM, total, 15)) + 8 <= esc_avail)
          k_scores<true, false>(sc, stage, tables, EscSrc<true>{stage + ST_ZERO, nullptr, esc_off}, flrow, rowoff, lane, Q);
        else
          k_scores<false, false>(sc, stage, tables, EscSrc<false>{nullptr, p.buf + (long)cur.mk * p.TS + SLOT_OVF_OFF, 0}, flrow, rowoff, lane, Q);
      } else raw_scores<false>(sc, p.raw + (long)(~cur.mk) * (T * D), nvalid, lane, Q);
    }
    // ---- the two halves' partial scores meet; the next tile's number and a failed wait travel with them
    uint8_t* slot = xch + par * XCH_PAR_BYTES;
    reinterpret_cast<float4*>(slot + hf * 512)[lane] = make_float4(sc[0], sc[1], sc[2], sc[3]);
    int* ctl = reinterpret_cast<int*>(slot + 1024);
    if (lane == 0) { if (hf == 0) ctl[0] = t1; if (!ok) ctl[1 + hf] = 1; }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    const float4 other = reinterpret_cast<const float4*>(slot + (hf ^ 1) * 512)[lane];
    sc[0] += other.x; sc[1] += other.y; sc[2] += other.z; sc[3] += other.w;
    t1 = ctl[0];
    const bool failed = (ctl[1] | ctl[2]) != 0;
    par ^= 1;
    if (failed) { if (lane == 0) atomicExch(p.err, 1); break; }                 // both warps of the pair see the same flags and leave together
    TileMeta nxt{0, 0};
    if (t1 < thi) { nxt = meta(t1); if (lane == 0) issue(ring_s + (stg ^ 1) * STAGE_BYTES, nxt); }
    PFrag P;
    if (nvalid == T) softmax_step<true>(A, sc, p.scale_log2, nvalid, lane, P);
    else softmax_step<false>(A, sc, p.scale_log2, nvalid, lane, P);
    if (!rawv) {
      if (esc_part(__shfl_sync(FULLM, total, 31)) + 8 <= esc_avail)
        v_accum<true, false>(A, stage, tables, EscSrc<true>{stage + ST_ZERO, nullptr, esc_off_v}, flrow, rowoff, lane, P);
      else
        v_accum<false, false>(A, stage, tables, EscSrc<false>{nullptr, p.buf + (long)cur.mv * p.TS + SLOT_OVF_OFF, 0}, flrow, rowoff, lane, P);
    } else raw_accum<false>(A, p.raw + (long)(~cur.mv) * (T * D), nvalid, lane, P);
    cur = nxt; stg ^= 1; tile = t1;
  }
  // ---- merge the warps of the CTA, half by half, and write one partial per virtual head (2 * query head + half)
  __syncthreads();
  constexpr int ACC_LD = D + 4;
  float* sh_m = reinterpret_cast<float*>(smem + TABLE256_BYTES);
  float* sh_l = sh_m + ATT_WARPS * 8;
  float* sh_acc = sh_l + ATT_WARPS * 8;
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) { A.l0 += __shfl_xor_sync(FULLM, A.l0, o); A.l1 += __shfl_xor_sync(FULLM, A.l1, o); }
  if (r == 0) { sh_m[warp * 8 + 2 * j] = A.m0; sh_l[warp * 8 + 2 * j] = A.l0; sh_m[warp * 8 + 2 * j + 1] = A.m1; sh_l[warp * 8 + 2 * j + 1] = A.l1; }
  if (2 * j < G) {
#pragma unroll
    for (int n = 0; n < 8; n++) {
      float* a0 = sh_acc + ((warp * 8 + 2 * j) * ACC_LD) + 16 * n + r;
      a0[0] = A.acc[n][0]; a0[ACC_LD] = A.acc[n][1]; a0[8] = A.acc[n][2]; a0[ACC_LD + 8] = A.acc[n][3];
    }
  }
  __syncthreads();
  const int d = tid & 127;
  for (int vg = tid >> 7; vg < 2 * G; vg += ATT_THREADS / 128) {
    const int g = vg >> 1, h2 = vg & 1;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < ATT_WARPS / 2; w++) M = fmaxf(M, sh_m[(2 * w + h2) * 8 + g]);
    float Lc = 0.f, Ac = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS / 2; w++) {
      const int ww = 2 * w + h2;
      const float mw = sh_m[ww * 8 + g];
      const float f = (mw == -CUDART_INF_F) ? 0.f : fast_exp2(mw - M);
      Lc += sh_l[ww * 8 + g] * f; Ac += sh_acc[(ww * 8 + g) * ACC_LD + d] * f;
    }
    const long vq = ((long)b * p.n_q + kvh * G + g) * 2 + h2, pidx = vq * p.nsplit + split;
    if (d == 0) { p.pm[pidx] = M * LN2; p.pl[pidx] = Lc; }                      // m in natural-log units, as gaac_combine expects
    p.pa[pidx * D + d] = Ac;
  }
}

// Second half of the cross-GPU exchange as a launch of its own (the attention kernel was launched push-only): wait until
// every rank's rows of this exchange have arrived in this GPU's receive buffer, merge them, and advance the exchange number.
// One CTA per query head.  A row that has not arrived after X_WAIT_LIMIT polls sets *err and the head comes back as zeros.
__global__ void __launch_bounds__(128) exchange_merge_kernel(unsigned long long* const* x_recv, int* epoch, int* ticket, int* err, int rank, int world,
                                                              long rows_cap, uint16_t* __restrict__ out, float* __restrict__ out_f32) {
  const long qh = blockIdx.x; const int d = threadIdx.x;
  asm volatile("griddepcontrol.wait;" ::: "memory");                   // resident early, runs after the attention kernel has completed
  asm volatile("griddepcontrol.launch_dependents;" ::);
  const int ep = __ldcg(epoch);                                         // advanced only after every CTA has taken its ticket
  float v;
  const int bad = !x_merge_rows(x_recv[rank] + (long)(ep & 1) * world * rows_cap * 130, world, rows_cap, qh, d, (u32)ep + 1u, v);
  const int any_bad = __syncthreads_or(bad);
  if (any_bad) { v = 0.f; if (d == 0) atomicExch(err, 1); }
  if (out) out[qh * D + d] = __bfloat16_as_ushort(__float2bfloat16(v));
  if (out_f32) out_f32[qh * D + d] = v;
  __syncthreads();
  if (d == 0) {
    __threadfence();
    if (atomicAdd(ticket, 1) == (int)gridDim.x - 1) { *ticket = 0; __threadfence(); atomicAdd(epoch, 1); }
  }
}

// Merge partials: pm, pl [n_heads, n_parts], pa [n_heads, n_parts, 128] (m in natural-log units).
__global__ void __launch_bounds__(128) combine_kernel(const float* __restrict__ pm, const float* __restrict__ pl, const float* __restrict__ pa,
                                                       int n_parts, uint16_t* __restrict__ out, float* __restrict__ out_f32) {
  const long qh = blockIdx.x; const int d = threadIdx.x;
  float M = -CUDART_INF_F;
  for (int s = 0; s < n_parts; s++) M = fmaxf(M, pm[qh * n_parts + s]);
  float L = 0.f, Ac = 0.f;
  for (int s = 0; s < n_parts; s++) {
    const float ms = pm[qh * n_parts + s];
    const float f = (ms == -CUDART_INF_F) ? 0.f : __expf(ms - M);
    L += pl[qh * n_parts + s] * f; Ac += pa[(qh * n_parts + s) * D + d] * f;
  }
  const float v = L > 0.f ? Ac / L : 0.f;
  if (out) out[qh * D + d] = __bfloat16_as_ushort(__float2bfloat16(v));
  if (out_f32) out_f32[qh * D + d] = v;
}

// The same merge over packed partials: parts [n_parts][n_heads][130] = (m in natural-log units, l, acc[128]) per head, the
// layout an all-gather of the ranks' gaac_decode_attn_partial outputs produces.
__global__ void __launch_bounds__(128) combine_parts_kernel(const float* __restrict__ parts, long n_heads, int n_parts,
                                                             uint16_t* __restrict__ out, float* __restrict__ out_f32) {
  const long qh = blockIdx.x; const int d = threadIdx.x;
  float M = -CUDART_INF_F;
  for (int s = 0; s < n_parts; s++) M = fmaxf(M, parts[(s * n_heads + qh) * 130]);
  float L = 0.f, Ac = 0.f;
  for (int s = 0; s < n_parts; s++) {
    const float* pp = parts + (s * n_heads + qh) * 130;
    const float ms = pp[0];
    const float f = (ms == -CUDART_INF_F) ? 0.f : __expf(ms - M);
    L += pp[1] * f; Ac += pp[2 + d] * f;
  }
  const float v = L > 0.f ? Ac / L : 0.f;
  if (out) out[qh * D + d] = __bfloat16_as_ushort(__float2bfloat16(v));
  if (out_f32) out_f32[qh * D + d] = v;
}

// Rows of a batch from the longest to the shortest (ties by index): entry k = {row, its token count}, k < B.  Entry B says whether
// the order is worth using: {1, -} when the shortest non-empty row has less than 7/8 of the longest row's tokens, else {0, -}
// (rows of about equal length keep the grid's own numbering, which costs nothing).  One CTA; every thread finds the place of its
// own row by counting the rows that come before it.
constexpr int ORDER_MAX_ROWS = 1024;
__global__ void __launch_bounds__(ORDER_MAX_ROWS) row_order_kernel(const int* __restrict__ seq_lens, const int* __restrict__ slot, int n_kv, int B,
                                                                   int2* __restrict__ order) {
  __shared__ int len_s[ORDER_MAX_ROWS];
  __shared__ int mx_s, mn_s;
  const int t = threadIdx.x;
  asm volatile("griddepcontrol.wait;" ::: "memory");                   // resident early behind the previous kernel, as the attention kernels are
  asm volatile("griddepcontrol.launch_dependents;" ::);
  if (t == 0) { mx_s = 0; mn_s = 0x7fffffff; }
  // paged layout: seq_lens[row]; slot layout: the tokens of the row's first head, seq_lens[slot[row] * n_kv] (0 for a padding row)
  if (t < B) len_s[t] = slot ? (slot[t] < 0 ? 0 : seq_lens[(long)slot[t] * n_kv]) : seq_lens[t];
  __syncthreads();
  if (t < B) {
    const int mine = len_s[t];
    atomicMax(&mx_s, mine);
    if (mine > 0) atomicMin(&mn_s, mine);
    int before = 0;
    for (int i = 0; i < B; i++) before += (len_s[i] > mine) || (len_s[i] == mine && i < t);
    order[before] = make_int2(t, mine);
  }
  __syncthreads();
  if (t == 0) order[B] = make_int2(mn_s < mx_s - (mx_s >> 3) ? 1 : 0, 0);
}

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
// Workspace = header | pm | pl | pa.  Header: the error word at byte 0, the split counters from byte 256.  The header has a
// fixed size for every B*n_q up to 16320, so the partials of a call never lie where the counters of a call of another shape
// do: a workspace zeroed once can be reused across batch sizes and split counts.
constexpr size_t WS_COUNTERS_OFF = 256, WS_MIN_HEADER = 64 << 10;
static size_t ws_header_bytes(int B, int n_q) { return std::max(WS_MIN_HEADER, WS_COUNTERS_OFF + align256(4 * (size_t)B * n_q)); }
static size_t ws_bytes_needed(int B, int n_q, int nsplit) {
  const size_t n = (size_t)B * n_q * nsplit;
  return ws_header_bytes(B, n_q) + align256(4 * n) * 2 + align256(4 * n * D) + align256(sizeof(int2) * ((size_t)B + 1));     // header | pm | pl | pa | row order
}
static int carve_workspace(void* ws, size_t ws_bytes, int B, int n_q, int nsplit, AttnParams& p) {
  const size_t n = (size_t)B * n_q * nsplit;
  if (!ws || ws_bytes < ws_bytes_needed(B, n_q, nsplit)) return GAAC_E_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(ws) & 15) return GAAC_E_ALIGN;
  uint8_t* w = (uint8_t*)ws;
  p.err = (int*)w; p.counters = (int*)(w + WS_COUNTERS_OFF); w += ws_header_bytes(B, n_q);
  p.pm = (float*)w; w += align256(4 * n);
  p.pl = (float*)w; w += align256(4 * n);
  p.pa = (float*)w; w += align256(4 * n * D);
  p.order_buf = (int2*)w;
  return GAAC_OK;
}

// Programmatic dependent launch of the attention and merge kernels (see gaac_set_launch_overlap); on unless switched off.
static int g_launch_overlap = 1;

static void launch_row_order(const int* seq_lens, const int* slot, int n_kv, int B, int2* order, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1); cfg.blockDim = dim3(ORDER_MAX_ROWS); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = g_launch_overlap;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, row_order_kernel, seq_lens, slot, n_kv, B, order) != cudaSuccess) cudaGetLastError();     // the attention launch that follows reports
}

template <bool PAGED, bool DUMP>
static int launch_attn(const AttnParams& p, cudaStream_t st) {
  cudaFuncSetAttribute(decode_attn_kernel<PAGED, DUMP>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.B * p.n_kv), (unsigned)p.nsplit); cfg.blockDim = dim3(ATT_THREADS);
  cfg.dynamicSmemBytes = ATT_SMEM; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = g_launch_overlap;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, decode_attn_kernel<PAGED, DUMP>, p) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  return launch_status();
}

static int sm_count_of_current_device() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!cached[dev]) { int n = 0; if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cached[dev] = n; else cudaGetLastError(); }
  return cached[dev];
}

static bool exchange_ok(const gaac_exchange* x) {
  return x && x->recv && x->epoch && x->ticket && x->err && x->world >= 1 && x->world <= 64 && x->rank >= 0 && x->rank < x->world && x->rows_cap > 0;
}

// What the slot-layout entry points differ in.
struct SlotOut {
  void* out = nullptr; float* out_f32 = nullptr; float* part = nullptr;
  const gaac_exchange* x = nullptr; bool fused = false;
  void* dump_k = nullptr; void* dump_v = nullptr; int64_t dump_S = 0;
};

static int slot_attn(const gaac_side* K, const gaac_side* V, const void* q, const int32_t* slot, int B, int n_q, int n_kv, const int32_t* seq_len,
                     int64_t S_uniform, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap, int n_base_rows, void* ws, size_t ws_bytes,
                     const SlotOut& o, void* stream) {
  const gaac_exchange* x = o.x;
  if (!K || !V || !q || (!o.out && !o.part && !x) || (x && o.fused && !o.out)) return GAAC_E_ARG;
  if (x && !exchange_ok(x)) return GAAC_E_ARG;
  if (B <= 0 || n_q <= 0 || n_kv <= 0 || nsplit <= 0 || nsplit > 1024 || S_pad <= 0 || S_pad % T || n_base_rows <= 0) return GAAC_E_ARG;
  if (!seq_len && (S_uniform < 0 || S_uniform > S_pad)) return GAAC_E_ARG;
  if (n_q % n_kv || n_q / n_kv < 1 || n_q / n_kv > 8) return GAAC_E_UNSUPPORTED;
  if (x && (int64_t)B * n_q > x->rows_cap) return GAAC_E_ARG;
  // fused exchange: a CTA per (row, kv head) waits for the other GPUs inside the kernel, so every CTA of the grid must be
  // resident at once (one CTA per SM); larger grids use the push + gaac_exchange_merge pair
  if (x && o.fused && (int64_t)B * n_kv * nsplit > sm_count_of_current_device()) return GAAC_E_UNSUPPORTED;
  for (const gaac_side* s : {K, V}) {
    if (!s->sm || !s->codes || !s->flags || !s->tile_off || !s->ovf || !s->head_start || !s->base3 || !s->base4 || s->ovf_bytes < 0) return GAAC_E_ARG;
    if (!aligned16(s->sm) || !aligned16(s->codes) || !aligned16(s->flags) || (reinterpret_cast<uintptr_t>(s->ovf) & 3)) return GAAC_E_ALIGN;
    if (tail_len && (!s->tail || (reinterpret_cast<uintptr_t>(s->tail) & 3))) return GAAC_E_ARG;
  }
  if (tail_len && tail_cap <= 0) return GAAC_E_ARG;
  if (reinterpret_cast<uintptr_t>(q) & 3) return GAAC_E_ALIGN;
  if ((o.dump_k || o.dump_v) && (!o.dump_k || !o.dump_v || o.dump_S <= 0 || (reinterpret_cast<uintptr_t>(o.dump_k) & 3) || (reinterpret_cast<uintptr_t>(o.dump_v) & 3))) return GAAC_E_ARG;
  AttnParams p{};
  p.K = *K; p.V = *V; p.slot = slot; p.seq_len = seq_len; p.S_uniform = (int)S_uniform; p.tail_len = tail_len; p.tail_cap = tail_cap; p.S_pad = S_pad; p.n_base_rows = n_base_rows;
  p.q = (const uint16_t*)q; p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.G = n_q / n_kv; p.scale_log2 = scale * LOG2E; p.nsplit = nsplit;
  p.out = (uint16_t*)o.out; p.out_f32 = o.out_f32; p.part = o.part;
  if (x) {
    p.x_recv = x->recv; p.x_epoch = x->epoch; p.x_ticket = x->ticket; p.x_err = x->err;
    p.x_rank = x->rank; p.x_world = x->world; p.x_rows_cap = x->rows_cap; p.x_fused = o.fused ? 1 : 0;
  }
  if (int e = carve_workspace(ws, ws_bytes, B, n_q, nsplit, p)) return e;
  if (o.dump_k) {
    p.dump_k = (uint16_t*)o.dump_k; p.dump_v = (uint16_t*)o.dump_v; p.dump_S = o.dump_S;
    return launch_attn<false, true>(p, (cudaStream_t)stream);
  }
  return launch_attn<false, false>(p, (cudaStream_t)stream);
}

static int paged_attn(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16, int B, int n_q, float scale,
                      int nsplit, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32, void* dump_k, void* dump_v, int64_t dump_S, void* stream) {
  if (!st || !bt || !seq_lens || !q_bf16 || !out_bf16 || !st->buf || !st->raw || !st->mt || !st->b3k || !st->b4k || !st->b3v || !st->b4v) return GAAC_E_ARG;
  if (B <= 0 || n_q <= 0 || st->n_kv <= 0 || nsplit <= 0 || nsplit > 1024 || bt_stride <= 0) return GAAC_E_ARG;
  if (n_q % st->n_kv || n_q / st->n_kv < 1 || n_q / st->n_kv > 8 || st->TS % 16 || st->TS != SLOT_OVF_OFF + st->ovf_slot) return GAAC_E_UNSUPPORTED;
  if (!aligned16(st->buf) || (reinterpret_cast<uintptr_t>(st->raw) & 3) || (reinterpret_cast<uintptr_t>(q_bf16) & 3)) return GAAC_E_ALIGN;
  if ((dump_k || dump_v) && (!dump_k || !dump_v || dump_S <= 0 || (reinterpret_cast<uintptr_t>(dump_k) & 3) || (reinterpret_cast<uintptr_t>(dump_v) & 3))) return GAAC_E_ARG;
  AttnParams p{};
  p.buf = st->buf; p.raw = (const uint16_t*)st->raw; p.mt = st->mt; p.bt = bt; p.bt_stride = bt_stride; p.TS = st->TS; p.ovf_slot = st->ovf_slot;
  p.b3k = st->b3k; p.b4k = st->b4k; p.b3v = st->b3v; p.b4v = st->b4v; p.seq_len = seq_lens;
  p.q = (const uint16_t*)q_bf16; p.B = B; p.n_q = n_q; p.n_kv = st->n_kv; p.G = n_q / st->n_kv; p.scale_log2 = scale * LOG2E; p.nsplit = nsplit;
  p.out = (uint16_t*)out_bf16; p.out_f32 = out_f32; p.part = nullptr;
  if (int e = carve_workspace(workspace, workspace_bytes, B, n_q, nsplit, p)) return e;
  if (dump_k) {
    p.dump_k = (uint16_t*)dump_k; p.dump_v = (uint16_t*)dump_v; p.dump_S = dump_S;
    return launch_attn<true, true>(p, (cudaStream_t)stream);
  }
  // ragged batches: CTAs are handed out longest row first (one small launch sorts the rows; its output is read by the attention
  // kernel after its dependency wait)
  if (B > 1 && B <= ORDER_MAX_ROWS && (int64_t)B * st->n_kv * nsplit > sm_count_of_current_device()) {
    launch_row_order(seq_lens, nullptr, 0, B, p.order_buf, (cudaStream_t)stream);
    p.row_order = p.order_buf;
  }
  return launch_attn<true, false>(p, (cudaStream_t)stream);
}

}  // namespace gaac

using namespace gaac;

extern "C" void gaac_set_launch_overlap(int enabled) { g_launch_overlap = enabled ? 1 : 0; }

extern "C" size_t gaac_attn_workspace_bytes(int B, int n_q, int nsplit) {
  if (B <= 0 || n_q <= 0 || nsplit <= 0) return 0;
  return ws_bytes_needed(B, n_q, nsplit);
}

extern "C" size_t gaac_attn_workspace_header_bytes(int B, int n_q) {
  if (B <= 0 || n_q <= 0) return 0;
  return ws_header_bytes(B, n_q);
}

extern "C" int gaac_decode_attn(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                                int n_base_rows, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32, void* stream) {
  if (!out_bf16 || !slot || !seq_len) return GAAC_E_ARG;
  SlotOut o; o.out = out_bf16; o.out_f32 = out_f32;
  return slot_attn(K, V, q_bf16, slot, B, n_q, n_kv, seq_len, 0, S_pad, scale, nsplit, tail_len, tail_cap, n_base_rows, workspace, workspace_bytes, o, stream);
}

extern "C" int gaac_decode_attn_pages(const gaac_side* K, const gaac_side* V, const void* q_bf16, int B, int n_q, int n_kv, int64_t S, int64_t S_pad,
                                      float scale, int nsplit, int n_base_rows, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32,
                                      float* part, const gaac_exchange* x, int fused, void* stream) {
  if ((out_bf16 != nullptr) + (part != nullptr) + (x != nullptr && !fused) != 1) return GAAC_E_ARG;      // exactly one destination
  SlotOut o; o.out = out_bf16; o.out_f32 = out_f32; o.part = part; o.x = x; o.fused = x && fused;
  return slot_attn(K, V, q_bf16, nullptr, B, n_q, n_kv, nullptr, S, S_pad, scale, nsplit, nullptr, 0, n_base_rows, workspace, workspace_bytes, o, stream);
}

extern "C" int gaac_decode_attn_partial(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                        const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                                        int n_base_rows, void* workspace, size_t workspace_bytes, float* part, void* stream) {
  if (!part || !slot || !seq_len) return GAAC_E_ARG;
  SlotOut o; o.part = part;
  return slot_attn(K, V, q_bf16, slot, B, n_q, n_kv, seq_len, 0, S_pad, scale, nsplit, tail_len, tail_cap, n_base_rows, workspace, workspace_bytes, o, stream);
}

extern "C" int gaac_combine(const float* pm, const float* pl, const float* pa, int64_t n_heads, int n_parts, void* out_bf16, float* out_f32, void* stream) {
  if (!pm || !pl || !pa || n_heads <= 0 || n_parts <= 0 || (!out_bf16 && !out_f32)) return GAAC_E_ARG;
  combine_kernel<<<(unsigned)n_heads, 128, 0, (cudaStream_t)stream>>>(pm, pl, pa, n_parts, (uint16_t*)out_bf16, out_f32);
  return launch_status();
}

extern "C" int gaac_decode_attn_push(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                     const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                                     int n_base_rows, void* workspace, size_t workspace_bytes, const gaac_exchange* x, void* stream) {
  if (!x || !slot || !seq_len) return GAAC_E_ARG;
  SlotOut o; o.x = x;
  return slot_attn(K, V, q_bf16, slot, B, n_q, n_kv, seq_len, 0, S_pad, scale, nsplit, tail_len, tail_cap, n_base_rows, workspace, workspace_bytes, o, stream);
}

extern "C" int gaac_decode_attn_exchange(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                         const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                                         int n_base_rows, void* workspace, size_t workspace_bytes, const gaac_exchange* x, void* out_bf16, float* out_f32,
                                         void* stream) {
  if (!x || !slot || !seq_len || !out_bf16) return GAAC_E_ARG;
  SlotOut o; o.x = x; o.fused = true; o.out = out_bf16; o.out_f32 = out_f32;
  return slot_attn(K, V, q_bf16, slot, B, n_q, n_kv, seq_len, 0, S_pad, scale, nsplit, tail_len, tail_cap, n_base_rows, workspace, workspace_bytes, o, stream);
}

extern "C" int gaac_exchange_merge(const gaac_exchange* x, int64_t n_heads, void* out_bf16, float* out_f32, void* stream) {
  if (!exchange_ok(x)) return GAAC_E_ARG;
  if (n_heads <= 0 || n_heads > x->rows_cap || (!out_bf16 && !out_f32)) return GAAC_E_ARG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)n_heads); cfg.blockDim = dim3(128); cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = g_launch_overlap;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, exchange_merge_kernel, x->recv, x->epoch, x->ticket, x->err, x->rank, x->world,
                         (long)x->rows_cap, (uint16_t*)out_bf16, out_f32) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  return launch_status();
}

extern "C" int gaac_combine_parts(const float* parts, int64_t n_heads, int n_parts, void* out_bf16, float* out_f32, void* stream) {
  if (!parts || n_heads <= 0 || n_parts <= 0 || (!out_bf16 && !out_f32)) return GAAC_E_ARG;
  combine_parts_kernel<<<(unsigned)n_heads, 128, 0, (cudaStream_t)stream>>>(parts, (long)n_heads, n_parts, (uint16_t*)out_bf16, out_f32);
  return launch_status();
}

extern "C" int gaac_paged_decode_attn(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16,
                                      int B, int n_q, float scale, int nsplit, void* workspace, size_t workspace_bytes,
                                      void* out_bf16, float* out_f32, void* stream) {
  return paged_attn(st, bt, bt_stride, seq_lens, q_bf16, B, n_q, scale, nsplit, workspace, workspace_bytes, out_bf16, out_f32, nullptr, nullptr, 0, stream);
}

extern "C" int gaac_paged_decode_attn256(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16,
                                         int B, int n_q, float scale, int nsplit, void* workspace, size_t workspace_bytes,
                                         void* out_bf16, float* out_f32, void* stream) {
  if (!st || !bt || !seq_lens || !q_bf16 || !out_bf16 || !st->buf || !st->raw || !st->mt || !st->b3k || !st->b4k || !st->b3v || !st->b4v) return GAAC_E_ARG;
  if (B <= 0 || n_q <= 0 || st->n_kv <= 0 || nsplit <= 0 || nsplit > 1024 || bt_stride <= 0) return GAAC_E_ARG;
  if (st->n_kv % 2) return GAAC_E_UNSUPPORTED;                                // half-heads come in pairs
  const int n_kv = st->n_kv / 2;                                              // 256-dim kv heads
  if (n_q % n_kv || n_q / n_kv < 1 || n_q / n_kv > 8 || st->TS % 16 || st->TS != SLOT_OVF_OFF + st->ovf_slot) return GAAC_E_UNSUPPORTED;
  if (!aligned16(st->buf) || (reinterpret_cast<uintptr_t>(st->raw) & 3) || (reinterpret_cast<uintptr_t>(q_bf16) & 3)) return GAAC_E_ALIGN;
  AttnParams p{};
  p.buf = st->buf; p.raw = (const uint16_t*)st->raw; p.mt = st->mt; p.bt = bt; p.bt_stride = bt_stride; p.TS = st->TS; p.ovf_slot = st->ovf_slot;
  p.b3k = st->b3k; p.b4k = st->b4k; p.b3v = st->b3v; p.b4v = st->b4v; p.seq_len = seq_lens;
  p.q = (const uint16_t*)q_bf16; p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.G = n_q / n_kv; p.scale_log2 = scale * LOG2E; p.nsplit = nsplit;
  if (int e = carve_workspace(workspace, workspace_bytes, B, 2 * n_q, nsplit, p)) return e;     // one partial per (query head, half)
  cudaFuncSetAttribute(paged256_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT256_SMEM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(B * n_kv), (unsigned)nsplit); cfg.blockDim = dim3(ATT_THREADS);
  cfg.dynamicSmemBytes = ATT256_SMEM; cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = g_launch_overlap;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, paged256_attn_kernel, p) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  // the halves' partials are laid out as 2 * B * n_q heads of 128 dims, which is out [B, n_q, 256] after the merge
  combine_kernel<<<(unsigned)(2 * B * n_q), 128, 0, (cudaStream_t)stream>>>(p.pm, p.pl, p.pa, nsplit, (uint16_t*)out_bf16, out_f32);
  return launch_status();
}

// ---- test hooks: the same kernels, instantiated so that every rebuilt BF16 fragment is also written to memory
extern "C" int gaac_debug_decode_attn_rebuild(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                              const int32_t* seq_len, int64_t S_uniform, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len,
                                              int tail_cap, int n_base_rows, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32,
                                              void* k_rebuilt, void* v_rebuilt, int64_t rebuilt_S, void* stream) {
  if (!out_bf16 || !k_rebuilt || !v_rebuilt) return GAAC_E_ARG;
  SlotOut o; o.out = out_bf16; o.out_f32 = out_f32; o.dump_k = k_rebuilt; o.dump_v = v_rebuilt; o.dump_S = rebuilt_S;
  return slot_attn(K, V, q_bf16, slot, B, n_q, n_kv, seq_len, S_uniform, S_pad, scale, nsplit, tail_len, tail_cap, n_base_rows, workspace, workspace_bytes, o, stream);
}

extern "C" int gaac_debug_paged_decode_attn_rebuild(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16,
                                                    int B, int n_q, float scale, int nsplit, void* workspace, size_t workspace_bytes, void* out_bf16,
                                                    float* out_f32, void* k_rebuilt, void* v_rebuilt, int64_t rebuilt_S, void* stream) {
  if (!k_rebuilt || !v_rebuilt) return GAAC_E_ARG;
  return paged_attn(st, bt, bt_stride, seq_lens, q_bf16, B, n_q, scale, nsplit, workspace, workspace_bytes, out_bf16, out_f32, k_rebuilt, v_rebuilt, rebuilt_S, stream);
}
