// Decode attention for callers that must not allocate device memory.
//
// Who that is: code that runs where an allocation is either illegal or unaffordable - a serving loop whose whole HBM budget
// was handed to the cache pool at start-up (a late cudaMalloc can simply fail there), a plugin host that forbids allocator
// calls on its hot path, or a caller that has no allocator of its own to hand out a workspace tensor.  The regular entry
// point (gaac_decode_attn) asks such a caller for a workspace; this one brings its own.
//
// The workspace (split partials + the per-head ticket counters of the fused kernel) lives in a file-scope device array of a
// fixed, modest size.  Every GPU that loads the library holds these bytes until the process exits.  All calls on a device
// share the array: it keeps the previous call's contents, the part that has to start at zero (the counters) is cleared on
// the stream in front of every launch (the error word in front of them is sticky and read with gaac_static_workspace_error), and two calls that overlap on the same GPU (different streams, or two host threads)
// race on it - callers serialise such calls themselves or use gaac_decode_attn with separate workspaces.
#include <mutex>
#include "gaac_api.cuh"

namespace {

constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;                   // 8 MiB: e.g. 32 query heads x 148 splits x 130 fp32 is 2.5 MB
static __device__ __align__(256) unsigned char g_scratch[STATIC_SCRATCH_BYTES];

// In host code `g_scratch` is only a handle for the runtime, not a device address: the address a kernel can use has to be
// asked for with cudaGetSymbolAddress, once per device, with that device current.
constexpr int MAX_DEVICES = 64;
void* g_scratch_ptr[MAX_DEVICES] = {};
std::mutex g_setup_mutex;

int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return GAAC_E_LAUNCH;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || !p) { cudaGetLastError(); return GAAC_E_LAUNCH; }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return GAAC_OK;
}

}  // namespace

extern "C" size_t gaac_static_workspace_bytes(void) { return STATIC_SCRATCH_BYTES; }

// Same arguments and results as gaac_decode_attn without the workspace pair.  Returns GAAC_E_WORKSPACE when
// gaac_attn_workspace_bytes(B, n_q, nsplit) exceeds gaac_static_workspace_bytes().  The first call on a device looks up the
// array's device address (cudaGetSymbolAddress); make that first call outside of any stream capture.
extern "C" int gaac_decode_attn_static(const gaac_side* K, const gaac_side* V, const void* q_bf16, const int32_t* slot, int B, int n_q, int n_kv,
                                       const int32_t* seq_len, int64_t S_pad, float scale, int nsplit, const int32_t* tail_len, int tail_cap,
                                       int n_base_rows, void* out_bf16, float* out_f32, void* stream) {
  if (B <= 0 || n_q <= 0 || nsplit <= 0) return GAAC_E_ARG;
  const size_t need = gaac_attn_workspace_bytes(B, n_q, nsplit);
  if (need == 0 || need > STATIC_SCRATCH_BYTES) return GAAC_E_WORKSPACE;
  void* ws = nullptr;
  if (int e = scratch_for_current_device(&ws)) return e;
  // The split counters (everything in the header behind its first 256 bytes) must start at zero whatever an earlier call left
  // behind.  The first 256 bytes hold the error word, which is sticky: it is left alone here so that a caller can still read
  // it with gaac_static_workspace_error after later calls.
  const size_t header = gaac_attn_workspace_header_bytes(B, n_q);
  if (cudaMemsetAsync((unsigned char*)ws + 256, 0, header - 256, (cudaStream_t)stream) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  return gaac_decode_attn(K, V, q_bf16, slot, B, n_q, n_kv, seq_len, S_pad, scale, nsplit, tail_len, tail_cap, n_base_rows,
                          ws, STATIC_SCRATCH_BYTES, out_bf16, out_f32, stream);
}

// The error word of the shared array on the current device: *err_host becomes 1 when a bounded wait inside one of the
// gaac_decode_attn_static calls made so far on this device ran out (the output of that call was not valid), else 0; with
// clear != 0 the word is reset afterwards.  Waits for `stream` (it copies four bytes to the host), so it is not for the hot
// path: call it where the caller synchronises anyway.
extern "C" int gaac_static_workspace_error(int32_t* err_host, int clear, void* stream) {
  if (!err_host) return GAAC_E_ARG;
  void* ws = nullptr;
  if (int e = scratch_for_current_device(&ws)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyAsync(err_host, ws, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  if (clear && cudaMemsetAsync(ws, 0, sizeof(int32_t), st) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  if (cudaStreamSynchronize(st) != cudaSuccess) { cudaGetLastError(); return GAAC_E_LAUNCH; }
  return GAAC_OK;
}
