// Host emulation of one warp encoding / rebuilding a GAAC tile with the SAME lane-level functions the CUDA kernels use
// (gaac_b200/csrc/gaac_tile.h).  The warp-level glue (tag table, row prefix sums) is replaced by plain loops.
// Built by the test-suite with g++ and driven through ctypes; checks the bit logic without a GPU.
#include <cstring>
#include "../../gaac_b200/csrc/gaac_tile.h"
using namespace gaac;

struct PtrEscH {
  const uint8_t* p;
  u32 byte(int pos) const { return p[pos]; }
  u64 bytes5(int pos) const { u64 w = 0; for (int i = 0; i < 5; i++) w |= (u64)p[pos + i] << (8 * i); return w; }
};
static int v_tok(int j, int t) { return 2 * j + (t & 1) + 8 * (t >> 1); }

extern "C" int emu_encode_tile(int kind_v, const uint16_t* x, int nvalid, const uint8_t* b3row, const uint8_t* b4row,
                               uint8_t* sm_out, uint8_t* cd_out, uint32_t* fl_out, uint8_t* esc_out) {
  uint8_t tag[16][16]; u64 escv[16][16];
  memset(tag, 0, sizeof tag); memset(escv, 0, sizeof escv);
  memset(sm_out, 0, 2048); memset(cd_out, 0, 768);
  for (int lane = 0; lane < 32; lane++) {
    int j = lane & 3, r = lane >> 2;
    if (!kind_v) {
      u32 b3w[8], b4w[8]; k_base_words(b3row, j, b3w); k_base_words(b4row, j, b4w);
      for (int o = 0; o < 2; o++) {
        int row = 8 * o + r; if (row >= nvalid) continue;
        u32 sm[8], cd[3], t8; u64 esc[4];
        encode_k_lane(x + row * 128, j, b3w, b4w, sm, cd, t8, esc);
        memcpy(sm_out + o * 1024 + 32 * lane, sm, 32); memcpy(cd_out + o * 384 + 12 * lane, cd, 12);
        for (int g = 0; g < 4; g++) { tag[row][4 * j + g] = (t8 >> (2 * g)) & 3; escv[row][4 * j + g] = esc[g]; }
      }
    } else {
      u32 b3w[4], b4w[4]; v_base_words(b3row, r, b3w); v_base_words(b4row, r, b4w);
      for (int t = 0; t < 4; t++) {
        int row = v_tok(j, t); if (row >= nvalid) continue;
        u32 sm[4], t4; u64 cd48, esc[2];
        encode_v_lane(x + row * 128, r, b3w, b4w, sm, cd48, t4, esc);
        memcpy(sm_out + 64 * lane + 16 * t, sm, 16); memcpy(cd_out + 24 * lane + 6 * t, &cd48, 6);
        for (int g = 0; g < 2; g++) { tag[row][2 * r + g] = (t4 >> (2 * g)) & 3; escv[row][2 * r + g] = esc[g]; }
      }
    }
  }
  int pos = 0;
  for (int row = 0; row < 16; row++) {
    u32 fl = 0;
    for (int g = 0; g < 16; g++) {
      fl |= (u32)tag[row][g] << (2 * g);
      int n = tag_esc_bytes(tag[row][g]);
      for (int i = 0; i < n; i++) esc_out[pos++] = (uint8_t)(escv[row][g] >> (8 * i));
    }
    fl_out[row] = fl;
  }
  return pos;
}

extern "C" void emu_decode_tile(int kind_v, const uint8_t* sm_in, const uint8_t* cd_in, const uint32_t* fl_in, const uint8_t* esc_in,
                                const uint8_t* b3row, const uint8_t* b4row, uint16_t* out) {
  int rowoff[16], acc = 0;
  for (int row = 0; row < 16; row++) { rowoff[row] = acc; acc += row_esc_bytes(fl_in[row]); }
  PtrEscH esc{esc_in};
  for (int lane = 0; lane < 32; lane++) {
    int j = lane & 3, r = lane >> 2;
    if (!kind_v) {
      u32 b3w[8], b4w[8]; k_base_words(b3row, j, b3w); k_base_words(b4row, j, b4w);
      for (int o = 0; o < 2; o++) {
        int row = 8 * o + r; u32 sm[8], cd[3];
        memcpy(sm, sm_in + o * 1024 + 32 * lane, 32); memcpy(cd, cd_in + o * 384 + 12 * lane, 12);
        u32 fl = fl_in[row]; int pos = rowoff[row] + esc_prefix(fl, 8 * j);
        for (int g = 0; g < 4; g++) {
          u32 o4[4];
          decode_group(sm[2 * g], sm[2 * g + 1], k_group_codes(cd, g), (fl >> (8 * j + 2 * g)) & 3u, pos, esc, b3w[2 * g], b3w[2 * g + 1], b4w[2 * g] - b3w[2 * g], b4w[2 * g + 1] - b3w[2 * g + 1], o4);
          for (int h = 0; h < 2; h++) {
            int s = 2 * g + h; uint16_t* p = out + row * 128 + 16 * s + 2 * j;
            p[0] = (uint16_t)o4[2 * h]; p[1] = (uint16_t)(o4[2 * h] >> 16); p[8] = (uint16_t)o4[2 * h + 1]; p[9] = (uint16_t)(o4[2 * h + 1] >> 16);
          }
        }
      }
    } else {
      u32 b3w[4], b4w[4]; v_base_words(b3row, r, b3w); v_base_words(b4row, r, b4w);
      u32 cd[6]; memcpy(cd, cd_in + 24 * lane, 24);
      for (int t = 0; t < 4; t++) {
        int row = v_tok(j, t); u32 sm[4]; memcpy(sm, sm_in + 64 * lane + 16 * t, 16);
        u32 fl = fl_in[row]; int pos = rowoff[row] + esc_prefix(fl, 4 * r);
        for (int g = 0; g < 2; g++) {
          u32 o4[4];
          decode_group(sm[2 * g], sm[2 * g + 1], v_group_codes(cd, t, g), (fl >> (4 * r + 2 * g)) & 3u, pos, esc, b3w[2 * g], b3w[2 * g + 1], b4w[2 * g] - b3w[2 * g], b4w[2 * g + 1] - b3w[2 * g + 1], o4);
          for (int h = 0; h < 2; h++) {
            int w = 2 * g + h; uint16_t* p = out + row * 128 + r;
            p[8 * (4 * w)] = (uint16_t)o4[2 * h]; p[8 * (4 * w + 1)] = (uint16_t)(o4[2 * h] >> 16);
            p[8 * (4 * w + 2)] = (uint16_t)o4[2 * h + 1]; p[8 * (4 * w + 3)] = (uint16_t)(o4[2 * h + 1] >> 16);
          }
        }
      }
    }
  }
}

// Same as emu_decode_tile through the table-driven group decoder of the fused attention kernel.
// esc_in must be 4-byte aligned and readable 8 bytes past its last escape byte.
extern "C" void emu_decode_tile_lut(int kind_v, const uint8_t* sm_in, const uint8_t* cd_in, const uint32_t* fl_in, const uint8_t* esc_in,
                                    const uint8_t* b3row, const uint8_t* b4row, uint16_t* out) {
  static u32x2 lutx[256]; static bool init = false;
  if (!init) { for (int i = 0; i < 256; i++) fill_lutx(lutx, i); init = true; }
  static const uint32_t zero_word = 0; const uint8_t* zero = reinterpret_cast<const uint8_t*>(&zero_word);
  int rowoff[16], acc = 0;
  for (int row = 0; row < 16; row++) { rowoff[row] = acc; acc += row_esc_bytes(fl_in[row]); }
  for (int lane = 0; lane < 32; lane++) {
    int j = lane & 3, r = lane >> 2;
    if (!kind_v) {
      u32 b3w[8], b4w[8]; k_base_words(b3row, j, b3w); k_base_words(b4row, j, b4w);
      for (int o = 0; o < 2; o++) {
        int row = 8 * o + r; u32 sm[8], cd[3];
        memcpy(sm, sm_in + o * 1024 + 32 * lane, 32); memcpy(cd, cd_in + o * 384 + 12 * lane, 12);
        u32 fl = fl_in[row]; int pos = rowoff[row] + esc_prefix(fl, 8 * j);
        for (int g = 0; g < 4; g++) {
          u32 o4[4]; u32x4 bw{b3w[2 * g], b3w[2 * g + 1], b4w[2 * g] - b3w[2 * g], b4w[2 * g + 1] - b3w[2 * g + 1]};
          decode_group_lut(sm[2 * g], sm[2 * g + 1], k_group_codes(cd, g), (fl >> (8 * j + 2 * g)) & 3u, pos, esc_in, zero, lutx, bw, o4);
          for (int h = 0; h < 2; h++) {
            int s = 2 * g + h; uint16_t* p = out + row * 128 + 16 * s + 2 * j;
            p[0] = (uint16_t)o4[2 * h]; p[1] = (uint16_t)(o4[2 * h] >> 16); p[8] = (uint16_t)o4[2 * h + 1]; p[9] = (uint16_t)(o4[2 * h + 1] >> 16);
          }
        }
      }
    } else {
      u32 b3w[4], b4w[4]; v_base_words(b3row, r, b3w); v_base_words(b4row, r, b4w);
      u32 cd[6]; memcpy(cd, cd_in + 24 * lane, 24);
      for (int t = 0; t < 4; t++) {
        int row = v_tok(j, t); u32 sm[4]; memcpy(sm, sm_in + 64 * lane + 16 * t, 16);
        u32 fl = fl_in[row]; int pos = rowoff[row] + esc_prefix(fl, 4 * r);
        for (int g = 0; g < 2; g++) {
          u32 o4[4]; u32x4 bw{b3w[2 * g], b3w[2 * g + 1], b4w[2 * g] - b3w[2 * g], b4w[2 * g + 1] - b3w[2 * g + 1]};
          decode_group_lut(sm[2 * g], sm[2 * g + 1], v_group_codes(cd, t, g), (fl >> (4 * r + 2 * g)) & 3u, pos, esc_in, zero, lutx, bw, o4);
          for (int h = 0; h < 2; h++) {
            int w = 2 * g + h; uint16_t* p = out + row * 128 + r;
            p[8 * (4 * w)] = (uint16_t)o4[2 * h]; p[8 * (4 * w + 1)] = (uint16_t)(o4[2 * h] >> 16);
            p[8 * (4 * w + 2)] = (uint16_t)o4[2 * h + 1]; p[8 * (4 * w + 3)] = (uint16_t)(o4[2 * h + 1] >> 16);
          }
        }
      }
    }
  }
}
