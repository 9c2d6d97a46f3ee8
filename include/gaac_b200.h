/* gaac_b200 — C ABI of the B200 (sm_100a) implementation of the GAAC KV-codec and compressed-KV decode attention.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its name ends in _host.  The library
 * allocates nothing: outputs and workspaces are caller-provided.  Every call enqueues work on `stream` (a cudaStream_t
 * passed as void*) and returns without synchronising, so a decode step stays CUDA-graph capturable.  Return value:
 * 0 on success, otherwise a GAAC_E_* code (see gaac_status_string); nothing is launched when an argument check fails.
 *
 * Each entry point names the interface of the reference implementation (Intelligent-Microsystems-Lab/GAAC) that it
 * replaces, as file:line of that project.
 */
#ifndef GAAC_B200_H
#define GAAC_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  GAAC_OK = 0,
  GAAC_E_ARG = 1,          /* null pointer, non-positive size, inconsistent sizes */
  GAAC_E_UNSUPPORTED = 2,  /* GQA group outside 1..8, head_dim != 128, tile stride not a multiple of 16 */
  GAAC_E_ALIGN = 3,        /* a buffer that must be 16-byte aligned is not */
  GAAC_E_LAUNCH = 4,       /* the CUDA runtime refused the launch (cudaGetLastError) */
  GAAC_E_WORKSPACE = 5     /* workspace too small */
};
#define GAAC_KIND_K 0
#define GAAC_KIND_V 1
#define GAAC_TILE_MAX_ESC 1280   /* worst-case escape bytes of a 16-token tile; stride of the encoder's scratch slots */

const char* gaac_status_string(int status);
/* ABI version of this header (bumped on any signature change). */
int gaac_abi_version(void);

/* ---------------------------------------------------------------------------------------------- block encoder */

/* Encode tiles 0..ceil(S/16)-1 of x [H, S_in, 128] bf16 into sm / codes / flags with a per-head token stride of S_pad;
 * the escape bytes of tile (h, t) go to slots + (h*ntiles + t)*GAAC_TILE_MAX_ESC and their count to tile_bytes[h*ntiles+t].
 * Head h uses base row bidx[h] when bidx != NULL, else h % n_kv.  Rows >= S of the last tile are stored as empty rows.
 * Replaces TileEncoder.encode_tiles / the Triton kernel _encode_tile (gaac/encoder.py:16-66, 94-102). */
int gaac_encode_tiles(const void* x_bf16, int64_t H, int64_t S, int64_t S_in, int64_t S_pad,
                      const uint8_t* base3, const uint8_t* base4, const int32_t* bidx, int n_kv, int kind,
                      uint8_t* sm, uint8_t* codes, int32_t* flags, uint8_t* slots, int32_t* tile_bytes, void* stream);

/* tile_off[h, t] = exclusive prefix of tile_bytes[h, :] (row stride tile_off_stride), head_bytes[h] = its sum (may be
 * NULL), then copy every scratch slot to ovf + head_start[h] + tile_off[h, t].  When head_start is NULL only the prefix
 * sums are produced (first pass, used to size ovf).  When ovf_off is non-NULL the per-row offsets within each head's escape
 * stream, ovf_off [H, S], are written as well (from flags [H, S_pad]).  Replaces TileEncoder.compact / _compact, the cumsum
 * between them (gaac/encoder.py:69-76, 104-109) and row_offsets (gaac/codec.py:221-225). */
int gaac_compact(const uint8_t* slots, const int32_t* tile_bytes, int64_t H, int64_t ntiles,
                 const int32_t* head_start, uint8_t* ovf, int32_t* tile_off, int64_t tile_off_stride, int32_t* head_bytes,
                 const int32_t* flags, int64_t S, int64_t S_pad, int32_t* ovf_off, void* stream);

/* TileEncoder.encode up to the point where the host must size the escape stream, in one call: gaac_encode_tiles, the prefix
 * sums of gaac_compact (tile_off [H, ntiles] contiguous, head_bytes [H]) and gaac_head_prefix (head_start [H+1]).  The caller
 * reads head_start[H], allocates ovf of that many bytes (+ padding) and finishes with gaac_compact_copy.  Same reference lines
 * as the three entry points it chains (gaac/encoder.py:94-121). */
int gaac_encode_begin(const void* x_bf16, int64_t H, int64_t S, int64_t S_in, int64_t S_pad,
                      const uint8_t* base3, const uint8_t* base4, const int32_t* bidx, int n_kv, int kind,
                      uint8_t* sm, uint8_t* codes, int32_t* flags, uint8_t* slots, int32_t* tile_bytes,
                      int32_t* tile_off, int32_t* head_bytes, int32_t* head_start, void* stream);

/* The copy half of gaac_compact with tile offsets that are already known: scratch slots -> ovf + head_start[h] + tile_off[h, t],
 * optionally the per-row offsets ovf_off [H, S], and zero_pad (0..32) zero bytes written behind the last head (the reference
 * allocates its stream with 8 bytes of over-read padding, gaac/encoder.py:121).  The copy is bounded, which lets a caller
 * allocate the stream before its size is known and so keep the whole encode free of host round trips: with ovf_cap > 0 nothing
 * is written at or beyond ovf + ovf_cap, with head_cap > 0 nothing of head h beyond head_start[h] + head_cap (zero_pad bytes of
 * read padding included in both); a tile that does not fit is skipped and bit 0 of *status (device int32, may be NULL) is set.  The
 * sizes in head_start / head_bytes are exact all the same, so the caller enlarges the buffer and repeats only this call (the
 * scratch slots are still valid).  Replaces _compact (gaac/encoder.py:69-76). */
int gaac_compact_copy(const uint8_t* slots, const int32_t* tile_bytes, int64_t H, int64_t ntiles, const int32_t* head_start, uint8_t* ovf,
                      const int32_t* tile_off, int64_t tile_off_stride, const int32_t* flags, int64_t S, int64_t S_pad, int32_t* ovf_off,
                      int zero_pad, int64_t ovf_cap, int64_t head_cap, int32_t* status, void* stream);

/* head_start[0..H] = exclusive prefix of head_bytes[0..H-1] (int32).  Replaces the head-level cumsum of
 * TileEncoder.encode (gaac/encoder.py:119-120). */
int gaac_head_prefix(const int32_t* head_bytes, int64_t H, int32_t* head_start, void* stream);

/* Bit-exact reconstruction of H heads x S tokens into out [H, S, 128] bf16.  ovf_off is not needed: row positions are
 * recomputed from the tag words.  Replaces Codec.decode (gaac/codec.py:186-218). */
int gaac_decode_page(const uint8_t* sm, const uint8_t* codes, const int32_t* flags, const int32_t* tile_off, int64_t tile_off_stride,
                     const uint8_t* ovf, const int32_t* head_start, const uint8_t* base3, const uint8_t* base4, const int32_t* bidx,
                     int n_kv, int kind, int64_t H, int64_t S, int64_t S_pad, void* out_bf16, void* stream);

/* hist[(c*256) + e] += number of rows of x [N, n_ch] bf16 whose channel c has exponent byte e (int64 counters, not
 * cleared here).  Replaces exponent_hist (gaac/codec.py:80-84). */
int gaac_exponent_hist(const void* x_bf16, int64_t N, int64_t n_ch, long long* hist, void* stream);

/* base3 / base4 [n_rows] = start of the densest 8- / 16-wide window of hist [n_rows, 256] (first maximum wins).
 * Replaces bases_from_hist (gaac/codec.py:70-77). */
int gaac_bases_from_hist(const long long* hist, int64_t n_rows, uint8_t* base3, uint8_t* base4, void* stream);

/* ---------------------------------------------------------------------------------------------- decode attention, slot layout */

/* One side (K or V) of a compressed cache in the slot layout (gaac/kv_cache.py:99-119; Page, gaac/codec.py:87-102). */
typedef struct {
  const uint8_t* sm;          /* [heads, S_pad*128] */
  const uint8_t* codes;       /* [heads, S_pad*48]  */
  const int32_t* flags;       /* [heads, S_pad]     */
  const int32_t* tile_off;    /* [heads, S_pad/16]  */
  const uint8_t* ovf;         /* escape stream */
  const int32_t* head_start;  /* [heads] offset of each head's escapes in ovf */
  int64_t ovf_bytes;          /* size of the ovf allocation (reads never go past it) */
  const uint8_t* base3;       /* [n_base_rows, 128] */
  const uint8_t* base4;
  const void* tail;           /* [heads, tail_cap, 128] bf16 raw tail, or NULL */
} gaac_side;

/* The attention and exchange-merge kernels are launched with programmatic stream serialisation allowed and begin with
 * griddepcontrol.wait: behind a kernel that signals early (these do) their CTAs become resident while that kernel is still
 * finishing, so consecutive attention layers overlap by a few microseconds; nothing is read or written before the wait returns.
 * enabled = 0 switches this off for later launches of the process (every launch then starts after its predecessor has finished
 * entirely, which is what a measurement of one launch's own duration wants); 1, the default, switches it back on.  Not
 * thread-safe against concurrent launches.  No counterpart in the reference. */
void gaac_set_launch_overlap(int enabled);

/* Bytes of workspace gaac_decode_attn / gaac_paged_decode_attn need for (B, n_q, nsplit), and the size of the header at its
 * start.  Workspace = header | split partials.  Header: an int32 error word at byte 0, the int32 split counters (one per row
 * and kv head) from byte 256.  The header must be zero on the first use; every call leaves the counters zero, so a workspace
 * is reusable as it is.  The header is 64 KiB for every B*n_q up to 16320, so calls of different shapes (batch size, head
 * count, split count) can share one workspace: no call's partials lie where another call's counters do.  Only a workspace that
 * has been used with B*n_q > 16320 must be zeroed again before it is used with a different B*n_q.  The error word is set to
 * 1 when a bounded wait of the kernel on its own asynchronous copies ran out (the output of that call is then not valid); it
 * is never cleared by the library and stays 0 in normal operation.  A workspace must be 16-byte aligned and must not be shared
 * by calls that overlap on the GPU. */
size_t gaac_attn_workspace_bytes(int B, int n_q, int nsplit);
size_t gaac_attn_workspace_header_bytes(int B, int n_q);

/* Fused decode attention over compressed K/V.  q [B, n_q, 128] bf16; batch row b reads cache head slot[b]*n_kv + kvh
 * (slot[b] < 0: padded row, output exactly 0); seq_len[cache head] compressed tokens; tail_len[cache head] raw tail tokens
 * (NULL when there is no tail).  nsplit >= 1 context splits per (row, kv head).  out [B, n_q, 128] bf16; when out_f32 is
 * non-NULL the un-rounded fp32 result is written there as well.  workspace: gaac_attn_workspace_bytes bytes with a zeroed
 * header (see above).  n_base_rows: rows of the base tables (cache head h uses row h % n_base_rows).  Replaces gaac_attn_launch = gaac_attn<G> + gaac_tail<G> + gaac_combine<128>
 * (gaac/kernel.py:48-326). */
int gaac_decode_attn(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                     const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                     int n_base_rows, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32, void* stream);

/* gaac_decode_attn for callers that cannot allocate device memory (a serving loop whose HBM was all handed to the cache
 * pool, a plugin host that forbids allocator calls on its hot path, a caller without an allocator of its own): same
 * arguments and results, but the workspace is a fixed 8 MiB array inside the library instead of a caller buffer.  No
 * counterpart in the reference, whose launcher allocates its partials with torch on every call (gaac/kernel.py:306-307).
 * Limits: gaac_attn_workspace_bytes(B, n_q, nsplit) must not exceed gaac_static_workspace_bytes(), else GAAC_E_WORKSPACE;
 * every GPU that loads the library holds the array until the process exits; all calls on a GPU share it, so calls that
 * overlap on one GPU race (serialise them, or use gaac_decode_attn with one workspace each).  The first call on a device
 * resolves the array's device address; make that call outside of any stream capture.
 * gaac_static_workspace_error copies the array's error word (see gaac_attn_workspace_bytes) of the current device to
 * *err_host, clears it afterwards when clear != 0, and waits for `stream`: the one way to learn that a bounded wait ran out in
 * an earlier gaac_decode_attn_static call; call it where the caller synchronises anyway. */
size_t gaac_static_workspace_bytes(void);
int gaac_static_workspace_error(int32_t* err_host, int clear, void* stream);
int gaac_decode_attn_static(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                            const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                            int n_base_rows, void* out_bf16, float* out_f32, void* stream);

/* Merge n_parts partial results per query head: pm, pl [n_heads, n_parts], pa [n_heads, n_parts, 128] fp32 ->
 * out [n_heads, 128] bf16 (and fp32 when out_f32 != NULL).  M = max m; L = sum l*exp(m-M); O = sum acc*exp(m-M)/L, 0 when
 * L <= 0; parts with m = -inf are skipped.  Replaces gaac_combine<128> (gaac/kernel.py:281-294); also the merge step of
 * the cross-GPU context split. */
int gaac_combine(const float* pm, const float* pl, const float* pa, int64_t n_heads, int n_parts, void* out_bf16, float* out_f32, void* stream);

/* gaac_combine over packed partials: parts [n_parts, n_heads, 130] fp32, each row (m, l, acc[128]) as written by
 * gaac_decode_attn_partial; this is the buffer an all-gather of the ranks' partials produces, so the cross-GPU merge is one
 * launch with no re-packing.  Same arithmetic as gaac_combine<128> (gaac/kernel.py:281-294). */
int gaac_combine_parts(const float* parts, int64_t n_heads, int n_parts, void* out_bf16, float* out_f32, void* stream);

/* As gaac_decode_attn, but stops after the per-(row, query head) merge of this GPU's splits and writes the un-normalised
 * partial (m, l, acc[128]) of every query head to part [B*n_q, 130] fp32 instead of the output (context split across
 * GPUs: the parts of all ranks are gathered and merged with gaac_combine).  No counterpart in the reference, which is
 * single-GPU; the partial has the layout of one split of gaac_attn<G> (gaac/kernel.py:206-216). */
int gaac_decode_attn_partial(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                             const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                             int n_base_rows, void* workspace, size_t workspace_bytes, float* part, void* stream);

/* Cross-GPU context split without a collective library on the data path: one process per GPU, every rank's receive buffer
 * mapped into every rank's address space (peer memory over NVLink).  No counterpart in the reference, which is single-GPU.
 *   recv[r]  : rank r's receive buffer, 2 * world * rows_cap * 130 entries of 8 bytes, zero before the first exchange (two
 *              exchanges deep, indexed by the parity of the exchange number, then by sending rank, then by query-head row
 *              b*n_q + head).  An entry = fp32 value in the low word, number of the exchange it belongs to in the high word,
 *              written with one 64-bit store and read with one 64-bit load: a reader that finds the expected number has the
 *              value that came with it, so no flag, fence or second trip over NVLink announces a row.  Numbers are compared for
 *              equality, so B and n_kv may change from one exchange to the next (within rows_cap), and an exchange that
 *              timed out leaves the following ones intact
 *   epoch, ticket, err : this rank's own device ints, zero before the first exchange; epoch = number of finished exchanges
 *              and must advance in step on all ranks (every rank makes the same sequence of calls); err becomes 1 when a
 *              wait ran out
 * recv is a DEVICE array of `world` pointers.  Buffers are two exchanges deep, which is enough as long as consecutive
 * exchanges use the same B, n_q and n_kv; ranks that change the shape synchronise with one another first. */
typedef struct {
  unsigned long long* const* recv;
  int32_t* epoch;
  int32_t* ticket;
  int32_t* err;
  int rank, world;
  int rows_cap;
} gaac_exchange;

/* gaac_decode_attn_partial whose last CTA of every (row, kv head) stores its partial rows straight into every rank's
 * receive buffer (64-bit stores over NVLink, each carrying the exchange number): the exchange rides on the attention
 * kernel's epilogue, there is no separate send.  Finish with gaac_exchange_merge on the same stream. */
int gaac_decode_attn_push(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                          const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                          int n_base_rows, void* workspace, size_t workspace_bytes, const gaac_exchange* x, void* stream);

/* Wait (bounded: about one second, then *err = 1 and a zero output) until the partials of all ranks for the current
 * exchange have arrived, merge them as gaac_combine does and advance the exchange number.  n_heads = B * n_q of the matching
 * gaac_decode_attn_push.  Launch it on the stream of the push, after it. */
int gaac_exchange_merge(const gaac_exchange* x, int64_t n_heads, void* out_bf16, float* out_f32, void* stream);

/* Push, wait and merge in ONE launch: the CTA that pushed the rows of a (row, kv head) group goes on to wait (same bound)
 * for the other ranks' rows of that group, merges them and writes out [B, n_q, 128] (out_f32 optional); the exchange number
 * advances when all groups are through.  Because CTAs wait for other GPUs inside the kernel, the whole grid must be resident
 * at once: B*n_kv*nsplit may not exceed the SM count (GAAC_E_UNSUPPORTED otherwise; use the pair above).  Every rank must
 * launch it for every exchange, one process per GPU: two "ranks" launched one after the other on ONE GPU would wait for each
 * other until the bound runs out. */
int gaac_decode_attn_exchange(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                              const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                              int n_base_rows, void* workspace, size_t workspace_bytes, const gaac_exchange* x, void* out_bf16, float* out_f32,
                              void* stream);

/* Decode attention over two Pages (all B*n_kv heads hold S tokens, row b reads heads b*n_kv .., no tail): the
 * `attention(q, kp, vp)` entry of the reference (gaac/kernel.py:345-359), which builds an identity slot map and a constant
 * length table for its launcher; here both are implied, so the kernel's prologue has no dependent table loads.  Exactly one
 * destination: out_bf16 (out_f32 optional) | part (as gaac_decode_attn_partial) | x with fused == 0 (as
 * gaac_decode_attn_push); x with fused != 0 and out_bf16 = gaac_decode_attn_exchange. */
int gaac_decode_attn_pages(const gaac_side* K, const gaac_side* V, const void* q_bf16, int B, int n_q, int n_kv, int64_t S, int64_t S_pad,
                           float scale, int nsplit, int n_base_rows, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32,
                           float* part, const gaac_exchange* x, int fused, void* stream);

/* ---------------------------------------------------------------------------------------------- slot cache (layout A) append */

/* Mutable side of the slot cache (gaac/kv_cache.py:99-119). */
typedef struct {
  uint8_t* sm; uint8_t* codes; int32_t* flags; int32_t* tile_off; uint8_t* ovf; int32_t* ovf_used; void* tail;
  const uint8_t* base3; const uint8_t* base4;
} gaac_store;

/* One new token per batch row: k_new/v_new [B, n_kv, 128] bf16, row b goes to cache head slot[b]*n_kv + kvh (slot < 0:
 * skipped).  Writes the token into the head's 16-token tail; when the tail fills, encodes it as tile seq_len/16, appends
 * its escapes at ovf + h*ovf_cap + ovf_used[h], sets tile_off and advances ovf_used; finally advances tail_len / seq_len.
 * A tile that would pass the head's token capacity, or whose escape bytes (+ 8 bytes of read padding) do not fit what is left of
 * the head's ovf_cap bytes, is not stored: nothing is written outside the head's share and the head's counters stay as they
 * were (the reference writes past the share in the second case, gaac/kv_cache.py:63-66; its callers avoid it with
 * check_capacity); the second case increments *err when err != NULL (device int32, e.g. polled with check_capacity).
 * Replaces _append_kv + _advance (gaac/kv_cache.py:22-96, 172-181). */
int gaac_append_kv(const gaac_store* K, const gaac_store* V, const void* k_new, const void* v_new, const int32_t* slot, int B, int n_kv,
                   int32_t* tail_len, int32_t* seq_len, int64_t S_cap, int64_t ovf_cap, int n_base_rows, int32_t* err, void* stream);

/* A whole prompt into one slot: k_tok / v_tok = the prompt's K and V as the model produces them, token-major: head h of token t
 * at x + t*row_stride + h*128 (bf16 elements; row_stride >= n_kv*128, rows 16-byte aligned), L tokens (L <= S_cap).  The
 * floor(L/16) whole tiles of every head of the slot are compressed straight into the store (tile 0 upward, the head's escape
 * bytes from offset 0 of its share), the L mod 16 remaining rows go into the raw tails, seq_len / tail_len / ovf_used of the
 * slot's heads are set: seven launches, no host synchronisation, no transposed copy of the input.
 * Replaces CompressedKVCache.prefill's device work (gaac/kv_cache.py:149-169: Triton encode per kind, torch prefix sums, the
 * scatter of the escape bytes, tail copy, counter updates).
 *   scratch: gaac_cache_prefill_scratch_bytes(L, n_kv) bytes of device memory, kept by the caller until a copy_only repeat is
 *     no longer needed.
 *   status: device int32[4], written by the call: [0] bit 0 set when some K head's escape bytes (+ 8 bytes of read padding) did
 *     not fit ovf_cap: the escape bytes of the tiles that did not fit were NOT written (nothing is written outside a head's
 *     share); tile_off and ovf_used are exact all the same; [1] = largest ovf_used among the slot's K heads; [2], [3]: same for V.
 *   copy_only != 0: after the caller has enlarged the escape streams (new K->ovf / V->ovf, new ovf_cap), repeat only the copy of
 *     the escape bytes from the scratch of the previous call with the same L and slot (k_tok / v_tok are not read and may be
 *     NULL); status[0] and status[2] are rewritten.
 * Base row of head slot*n_kv + h: (slot*n_kv + h) % n_base_rows, as in gaac_append_kv. */
size_t gaac_cache_prefill_scratch_bytes(int64_t L, int n_kv);
int gaac_cache_prefill(const gaac_store* K, const gaac_store* V, const void* k_tok, const void* v_tok, int64_t L, int64_t row_stride, int slot,
                       int n_kv, int32_t* tail_len, int32_t* seq_len, int64_t S_cap, int64_t ovf_cap, int n_base_rows, uint8_t* scratch,
                       size_t scratch_bytes, int32_t* status, int copy_only, void* stream);

/* ---------------------------------------------------------------------------------------------- paged layout (layout B) */

/* Paged store state of one layer (gaac/vllm/store.py:177-203).  Tile slot p = block*(2*n_kv) + 2*kvh + kind lives at
 * buf + p*TS: [0,2048) sign/mantissa, [2048,2816) codes, [2816,2880) 16 tag words, [2880,TS) escapes.
 * mt[p] == p: compressed in its slot; mt[p] == ~r: raw bf16 tile r of `raw` [raw_tiles,16,128]. */
typedef struct {
  uint8_t* buf; void* raw; int32_t* mt; int32_t* stack; int32_t* top; int32_t* err;
  const uint8_t* b3k; const uint8_t* b4k; const uint8_t* b3v; const uint8_t* b4v;
  int n_kv; int TS; int ovf_slot;
} gaac_paged;

/* Store this step's new rows.  key/value: [num_tokens, n_kv, 128] bf16 with row strides k_stride/v_stride (elements);
 * ent [E,4] = (block, first row in key/value, offset in block, rows); block < 0: inactive entry.  freeq [E*2*n_kv] scratch.
 * Filling blocks go to a raw tile (popped from the free stack on first touch); a block completed by this step is
 * compressed into its slot when its escapes fit ovf_slot (its raw tile is queued in freeq and pushed back), else kept
 * raw.  A failed pop increments *err.  Replaces _store_tiles + _free_tiles (gaac/vllm/store.py:22-114, 204-213). */
int gaac_paged_store(const gaac_paged* st, const void* key, const void* value, int64_t k_stride, int64_t v_stride,
                     const int32_t* ent, int E, int32_t* freeq, void* stream);

/* Give the raw tiles of freed blocks back and reset their mode-table entries.  Replaces _release_blocks
 * (gaac/vllm/store.py:166-174). */
int gaac_paged_release(const gaac_paged* st, const int32_t* blocks, int F, void* stream);

/* Expand blocks to bf16 rows of flat scratch tensors sk/sv [rows, n_kv, 128] (row stride in elements); pairs [P,3] =
 * (block, first scratch row, valid rows).  Replaces _decode_tiles (gaac/vllm/store.py:117-163). */
int gaac_paged_decode_blocks(const gaac_paged* st, const int32_t* pairs, int P, void* sk, void* sv, int64_t row_stride, void* stream);

/* Fused decode attention over the paged buffer: q [B, n_q, 128] bf16, out [B, n_q*128] bf16, bt [B, bt_stride] block
 * table, seq_lens [B] tokens per sequence (including the filling block).  Replaces gaac_vpaged_launch = gaac_vpaged<G> +
 * gaac_combine2<128> (gaac/vllm/paged_kernel.py:42-276).  When 1 < B <= 1024 and B*n_kv*nsplit exceeds the SM count a one-CTA
 * launch in front of the attention kernel sorts the rows by length, and the CTAs are handed out longest row first. */
int gaac_paged_decode_attn(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16,
                           int B, int n_q, float scale, int nsplit, void* workspace, size_t workspace_bytes,
                           void* out_bf16, float* out_f32, void* stream);

/* The same for head_dim 256: a 256-dim head is stored as two 128-dim half-heads in neighbouring tile slots, each with its own
 * bases, so the store, the block decoder and the bases all see 2 * (256-dim kv heads) half-heads: st->n_kv is that number of
 * HALF-heads (even), as for gaac_paged_store; the base tables have st->n_kv rows.  q [B, n_q, 256] bf16, out [B, n_q*256] bf16
 * (out_f32 optional), n_q a multiple of st->n_kv / 2 with group size 1..8.  workspace: gaac_attn_workspace_bytes(B, 2 * n_q,
 * nsplit) bytes.  Two launches (attention over warp pairs, then the split merge).  Replaces gaac_vpaged256_launch =
 * gaac_vpaged256<G> + gaac_combine2 (gaac/vllm/paged_kernel256.py:40-283, 299-305). */
int gaac_paged_decode_attn256(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16,
                              int B, int n_q, float scale, int nsplit, void* workspace, size_t workspace_bytes,
                              void* out_bf16, float* out_f32, void* stream);

/* ---------------------------------------------------------------------------------------------- test hooks */

/* gaac_decode_attn / gaac_paged_decode_attn compiled so that every BF16 fragment word the kernel rebuilds on its way to the
 * tensor cores is also written out: k_rebuilt / v_rebuilt [B*n_kv, rebuilt_S, 128] bf16, row t of (row b, kv head) = token t
 * of that head (compressed tiles, raw tiles, the filling block and the slot layout's tail behind the compressed tokens);
 * rows the kernel never reads are left untouched.  Same arguments otherwise (slot and seq_len may be NULL with S_uniform as
 * in gaac_decode_attn_pages), same attention output.  For tests: the rebuild inside the fused kernel (gaac/kernel.py:24-46,
 * 96-135 in the reference) is otherwise visible only through a softmax-weighted sum.  Slower than the regular entry. */
int gaac_debug_decode_attn_rebuild(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                   const int32_t* seq_len, int64_t S_uniform, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len,
                                   int tail_cap, int n_base_rows, void* workspace, size_t workspace_bytes, void* out_bf16, float* out_f32,
                                   void* k_rebuilt, void* v_rebuilt, int64_t rebuilt_S, void* stream);
int gaac_debug_paged_decode_attn_rebuild(const gaac_paged* st, const int32_t* bt, int64_t bt_stride, const int32_t* seq_lens, const void* q_bf16,
                                         int B, int n_q, float scale, int nsplit, void* workspace, size_t workspace_bytes, void* out_bf16,
                                         float* out_f32, void* k_rebuilt, void* v_rebuilt, int64_t rebuilt_S, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GAAC_B200_H */
