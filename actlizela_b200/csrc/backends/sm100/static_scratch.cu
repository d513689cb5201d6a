// Forward entry point that needs no allocator: the WY-factor workspace lives in a fixed device
// array that is part of this library's image.
//
// Who this is for: callers that are handed device pointers for their inputs and outputs but
// have no way to obtain scratch memory themselves, for example a plugin running inside a host
// framework that owns every allocation and forbids cudaMalloc on its threads, or a real-time
// loop in which an allocation (and the implicit device synchronisation it can cause) is not
// acceptable.  They still pass q, k, v, g, beta, the optional initial state, the output and the
// optional final state; only the scratch that the prepare kernel fills and the chunk walk reads
// comes from here.
//
// Limits and rules, all of which the caller must know:
//   * The array holds ACTLIZE_LA_SM100_STATIC_SCRATCH_MAX_BLOCKS blocks, one block per
//     (batch, value head, 64-token chunk): B * Hv * ceil(T / 64) must not exceed it.  A larger
//     geometry is refused with ACTLIZE_LA_SM100_ERROR_SCRATCH_TOO_SMALL and a one-line message on
//     stderr; nothing is launched.  Every GPU on which the library is loaded keeps the array
//     (about 4.6 MiB) until the process exits.
//   * The first call on a device performs a one-time set-up on that device (kernel attributes and
//     the look-up of the array's device address).  Make that first call before any stream capture.
//   * All calls share the one array and it keeps the previous call's contents.  Nothing in it has to
//     start at zero: the prepare kernel rewrites every element the walk reads.  Two calls that
//     overlap on the GPU (different streams, or graphs replayed concurrently) race on it; run them
//     one after the other.
//   * No cudaMalloc, cudaFree or allocating library routine is reached from this entry point.
#include "actlize_la_sm100.h"
#include "gdn_common.cuh"

#include <climits>
#include <cstdio>
#include <mutex>

namespace gdn_sm100 {
namespace {

constexpr long long kStaticBlocks = ACTLIZE_LA_SM100_STATIC_SCRATCH_MAX_BLOCKS;
constexpr long long kStaticBytes = kStaticBlocks * kBlockBytes;

// In host code this name is only a handle for the runtime; the address a kernel may use is the
// one cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};

// One-time set-up for the current device; returns a cudaError_t value.  The set-up cannot run while `stream` is
// being captured (it configures kernels and looks up a symbol address): a first call made inside a capture is
// refused with cudaErrorStreamCaptureUnsupported instead of breaking the capture.
int scratch_for_current_device(void** address, cudaStream_t stream) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return int(e);
  if (device < 0 || device >= kMaxDevices) return int(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[device]) {
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
      std::fprintf(stderr, "actlize_la_sm100_forward_static_scratch: the first call on a device sets the library up and "
                           "must be made before stream capture begins\n");
      return int(cudaErrorStreamCaptureUnsupported);
    }
    if (int rc = actlize_la_sm100_configure()) return rc;
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return int(e);
    if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255)) return int(cudaErrorInvalidSymbol);
    g_scratch_address[device] = ptr;
  }
  *address = g_scratch_address[device];
  return 0;
}

}  // namespace
}  // namespace gdn_sm100

using namespace gdn_sm100;

extern "C" int actlize_la_sm100_forward_static_scratch(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial, void* output, float* final_state,
    int b, int t, int hk, int hv, int gate_fp32, int config, void* stream) {
  if (b <= 0 || t <= 0 || hk <= 0 || hv <= 0 || hv % hk) return int(cudaErrorInvalidValue);
  const long long blocks = (long long)b * hv * ((t + kChunk - 1LL) / kChunk);
  if (blocks > kStaticBlocks) {
    std::fprintf(stderr,
                 "actlize_la_sm100_forward_static_scratch: B*Hv*ceil(T/64) = %lld blocks exceed the %lld "
                 "blocks of the built-in scratch array; use actlize_la_sm100_forward_prepared with a "
                 "caller-owned workspace\n", blocks, kStaticBlocks);
    return ACTLIZE_LA_SM100_ERROR_SCRATCH_TOO_SMALL;
  }
  void* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch, static_cast<cudaStream_t>(stream))) return rc;
  // the built-in array has no room for the carry state of a segmented walk: always one sequence segment here
  // (kernel family, stage and walk bits and the parallel sub-segment count pass through)
  return actlize_la_sm100_forward_prepared(q, k, v, g, beta, initial, output, final_state, scratch,
                                           kStaticBytes, b, t, hk, hv, gate_fp32, config & ~0xff00, stream);
}
