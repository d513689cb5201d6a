// extern "C" boundary of the cuda_sm100 backend (declared in include/actlize_la_sm100.h).
// Argument checking mirrors the reference's C launchers (csrc/backends/ppu10/launch.cu:57-65,
// csrc/backends/ppu15/bindings.cpp:28-31): reject null/ill-shaped input with an error code,
// guard the grid-size products, never throw, never allocate, never synchronise.
#include "actlize_la_sm100.h"
#include "gdn_common.cuh"

#include <climits>
#include <vector>

namespace gdn_sm100 {
namespace {

#include "sm100_policy_table.inc"   // generated from sm100_policy.json by the builder

bool geometry_ok(int b, int t, int hk, int hv) {
  if (b <= 0 || t <= 0 || hk <= 0 || hv <= 0 || hv % hk) return false;
  if (hk > INT_MAX / kDim || hv > INT_MAX / kDim) return false;
  const long long chunks = (t + kChunk - 1) / kChunk;
  const long long heads = (long long)b * hv;
  if (heads > INT_MAX / 8 || heads * chunks > INT_MAX / kDim) return false;     // flattened grids, 32-bit TMA rows
  if ((long long)b * t * hv * kDim > (1LL << 40)) return false;
  return true;
}

// Bits 4 and 5 of `config` restrict a call to one stage (per-kernel timing and diagnosis):
// 0x10 = prepare stage only, 0x20 = walk stage only (the workspace must already hold the
// factors of the same inputs).
// Bits 8..15 hold the number of sequence segments (0 or 1 = one): the prepare kernels of later
// segments then run next to the walk of earlier ones (tcgen05 configuration only).
// Bits 6 and 7 modify a walk-only call of the tcgen05 configuration (sequence-parallel scheme):
// 0x40 = treat U as zero (state-transition pass), 0x80 = stop each (batch, value head) walk once the decay
// accumulated since its start is below exp(-40) (no final state is written then).
// Bit 20 (0x100000) makes a walk-only call of the tcgen05 configuration the OFFSET pass of that scheme: per (batch,
// value head) only the shortest suffix of the sequence whose decay is below exp(-40) is walked, from a zero state,
// no output row is written, and `final_state` receives the state the sequence ends in from a zero (or, to exp(-40),
// any) incoming state; a head without such a suffix is walked whole.
// Bit 21 (0x200000) is the PAIR pass: the offset pass and the transition pass (0x40 from an identity state the kernel
// makes itself) in one launch, two CTAs per (batch, value head); `final_state` then points at the block
// [2][B][Hv][128][128] = (transition matrices, offsets), `initial` is not read, and `output` is scratch the
// transition CTAs may write.
// Bits 16..19 hold the number of parallel sub-segments of the tcgen05 walk (0 or 1 = off, at most 8): every
// (batch, value head) walk of a launch is cut into that many pieces walked by as many CTAs at the same time
// (walk_umma_kernel); needs the tcgen05 prepare stage, which records the per-chunk contraction flag the split relies on.
constexpr int kStageMask = 0x30, kPrepareOnly = 0x10, kWalkOnly = 0x20, kSegmentShift = 8, kMaxSegments = 16;
constexpr int kWalkFlagMask = 0xc0, kHomogeneousBit = 0x40, kUntilDecayedBit = 0x80;
constexpr int kParallelShift = 16, kMaxParallel = 8, kOffsetTailBit = 0x100000, kPairBit = 0x200000;
bool config_ok(int config) {
  const int segments = (config >> kSegmentShift) & 0xff, parallel = (config >> kParallelShift) & 0xf;
  if (config < 0 || (config & 0xf) > 3 ||
      (config & ~(kStageMask | kWalkFlagMask | 0xf | (0xff << kSegmentShift) | (0xf << kParallelShift) | kOffsetTailBit | kPairBit)) != 0)
    return false;
  if ((config & kOffsetTailBit) && (config & ~kOffsetTailBit) != (1 | kWalkOnly)) return false;
  if ((config & kPairBit) && (config & ~kPairBit) != (1 | kWalkOnly)) return false;
  if ((config & kWalkFlagMask) && ((config & 0xf) != 1 || (config & kStageMask) != kWalkOnly)) return false;
  if (parallel > kMaxParallel || (parallel > 1 && ((config & 0xf) != 1 || (config & kWalkFlagMask)))) return false;
  return (config & kStageMask) != kStageMask && segments <= kMaxSegments;
}
// parallel sub-segments for a launch that walks `chunks` chunks per (batch, value head)
int parallel_of(int config, int chunks) {
  const int parallel = (config >> kParallelShift) & 0xf;
  return parallel < 2 ? 1 : (parallel > chunks ? chunks : parallel);
}
int segments_of(int config, const Geometry& geo) {
  int segments = (config >> kSegmentShift) & 0xff;
  if ((config & 0xf) != 1 || (config & kStageMask) || segments < 2) return 1;
  const int chunks = geo.chunks();
  return segments > chunks ? chunks : segments;
}

// Second stream and events of the segmented forward, created by configure() for the current device.
struct SegmentStreams {
  cudaStream_t walk = nullptr;                    // high priority: the sequential chunk walks (host-buffer entry)
  cudaStream_t prepare = nullptr;                 // low priority: prepare kernels of the segments behind the first
  cudaStream_t copy_in = nullptr, copy_out = nullptr;   // host-buffer entry: transfers next to compute
  cudaEvent_t prepared[kMaxSegments] = {};
  cudaEvent_t arrived[kMaxSegments] = {};         // inputs of a segment are on the device
  cudaEvent_t walked[kMaxSegments] = {};          // a segment's output tile rows are complete
  cudaEvent_t done = nullptr, start = nullptr, copied = nullptr;
};
SegmentStreams g_streams[64];

int create_segment_streams() {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return int(e);
  if (device < 0 || device >= 64) return int(cudaErrorInvalidDevice);
  SegmentStreams& ss = g_streams[device];
  if (ss.walk) return 0;
  int least = 0, greatest = 0;
  if ((e = cudaDeviceGetStreamPriorityRange(&least, &greatest)) != cudaSuccess) return int(e);
  if ((e = cudaStreamCreateWithPriority(&ss.walk, cudaStreamNonBlocking, greatest)) != cudaSuccess) return int(e);
  if ((e = cudaStreamCreateWithPriority(&ss.prepare, cudaStreamNonBlocking, least)) != cudaSuccess) return int(e);
  if ((e = cudaStreamCreateWithFlags(&ss.copy_in, cudaStreamNonBlocking)) != cudaSuccess) return int(e);
  if ((e = cudaStreamCreateWithFlags(&ss.copy_out, cudaStreamNonBlocking)) != cudaSuccess) return int(e);
  for (int i = 0; i < kMaxSegments; ++i) {
    if ((e = cudaEventCreateWithFlags(&ss.prepared[i], cudaEventDisableTiming)) != cudaSuccess) return int(e);
    if ((e = cudaEventCreateWithFlags(&ss.arrived[i], cudaEventDisableTiming)) != cudaSuccess) return int(e);
    if ((e = cudaEventCreateWithFlags(&ss.walked[i], cudaEventDisableTiming)) != cudaSuccess) return int(e);
  }
  if ((e = cudaEventCreateWithFlags(&ss.start, cudaEventDisableTiming)) != cudaSuccess) return int(e);
  if ((e = cudaEventCreateWithFlags(&ss.copied, cudaEventDisableTiming)) != cudaSuccess) return int(e);
  return int(cudaEventCreateWithFlags(&ss.done, cudaEventDisableTiming));
}
// bit 0: prepare stage uses tcgen05 (1) or CUDA cores (0); configuration ids:
// 0 = simt/simt, 1 = umma/umma, 2 = simt prepare + umma walk, 3 = umma prepare + simt walk
bool prepare_is_umma(int config) { return (config & 0xf) == 1 || (config & 0xf) == 3; }
bool walk_is_umma(int config) { return (config & 0xf) == 1 || (config & 0xf) == 2; }
int launch_prepare_tc(int, const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  return in.mixed ? launch_prepare_fused(in, geo, ws, stream) : launch_prepare_umma(in, geo, ws, stream);
}
int launch_walk_tc(int, const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  return launch_walk_umma(in, geo, ws, stream);
}

// Offsets table of the packed mode from DEVICE offsets: cu_seqlens[0..n] (forced into 0 <= ... <= total and
// non-decreasing, so that no later index can leave the tensors) followed by the chunk prefix.
__global__ void varlen_table_kernel(const int* __restrict__ cu_seqlens, int n_seqs, int total, int* __restrict__ table) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int chunks = 0, previous = 0;
  table[0] = 0;
  table[n_seqs + 1] = 0;
  for (int i = 1; i <= n_seqs; ++i) {
    int at = cu_seqlens[i];
    at = at < previous ? previous : (at > total ? total : at);
    chunks += (at - previous + kChunk - 1) / kChunk;
    table[i] = at;
    table[n_seqs + 1 + i] = chunks;
    previous = at;
  }
}

// One affine step of a 128x128 state block, out = M @ S + b, by the 256 threads of a CTA (each 64 outputs).
// `s_in` and `s_out` may be the same block: every read of s_in is finished before the first write.
__device__ void affine_step(const float* m, const float* off, const float* s_in, float* s_out,
                            float (*tile_m)[129], float (*tile_s)[128]) {
  const int col = threadIdx.x % kDim, rhalf = threadIdx.x / kDim;
  const long long base = 0;
  {
    // a transition matrix of exact zeros (a segment that forgets its incoming state) leaves out = b
    bool nonzero = false;
    const float4* m4 = reinterpret_cast<const float4*>(m + base);
    for (int e = threadIdx.x; e < kDim * kDim / 4; e += blockDim.x) {
      const float4 x = m4[e];
      nonzero |= (x.x != 0.f) | (x.y != 0.f) | (x.z != 0.f) | (x.w != 0.f);
    }
    if (!__syncthreads_or(nonzero)) {
      const float4* b4 = reinterpret_cast<const float4*>(off + base);
      float4* o4 = reinterpret_cast<float4*>(s_out + base);
      for (int e = threadIdx.x; e < kDim * kDim / 4; e += blockDim.x) o4[e] = b4[e];
      return;
    }
  }
  float acc[64];
#pragma unroll
  for (int r = 0; r < 64; ++r) acc[r] = off[base + (rhalf * 64 + r) * kDim + col];
  for (int k0 = 0; k0 < kDim; k0 += 32) {
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * kDim; e += blockDim.x) {
      tile_m[e % 32][e / 32] = m[base + (e / 32) * kDim + k0 + e % 32];   // M[row][k0+kk]
      tile_s[e / kDim][e % kDim] = s_in[base + (k0 + e / kDim) * kDim + e % kDim];
    }
    __syncthreads();
    for (int kk = 0; kk < 32; ++kk) {
      const float sv = tile_s[kk][col];
#pragma unroll
      for (int r = 0; r < 64; ++r) acc[r] = fmaf(tile_m[kk][rhalf * 64 + r], sv, acc[r]);
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 64; ++r) s_out[base + (rhalf * 64 + r) * kDim + col] = acc[r];
}

__global__ void apply_transition_kernel(const float* __restrict__ m, const float* __restrict__ off,
                                        const float* __restrict__ s_in, float* __restrict__ s_out) {
  __shared__ float tile_m[32][129];
  __shared__ float tile_s[32][128];
  const long long base = (long long)blockIdx.x * kDim * kDim;
  affine_step(m + base, off + base, s_in + base, s_out + base, tile_m, tile_s);
}

// Exclusive scan of a rank's incoming state in one launch: `pairs` holds the (M_j, b_j) of the n earlier ranks as
// [n][2][blocks][128][128] (M_0 is unused: rank 0 contributes its true outgoing state as b_0);
// incoming = fold_j (M_j * incoming + b_j); optionally outgoing = my_m * incoming + my_b.  One CTA per block.
// The result is the same as folding from pair 0 on: a zero M_j makes everything before it irrelevant.
__global__ void fold_transitions_kernel(const float* __restrict__ pairs, int n, int blocks,
                                        float* __restrict__ incoming, float* __restrict__ outgoing,
                                        const float* __restrict__ my_m, const float* __restrict__ my_b) {
  __shared__ float tile_m[32][129];
  __shared__ float tile_s[32][128];
  const long long block = kDim * kDim, base = (long long)blockIdx.x * block;
  float* state = incoming + base;
  // the last pair whose transition is exactly zero forgets everything in front of it: the scan starts at its offset
  int start = 0;
  for (int j = n - 1; j >= 1; --j) {
    const float4* m4 = reinterpret_cast<const float4*>(pairs + (2LL * j * blocks) * block + base);
    bool nonzero = false;
    for (int e = threadIdx.x; e < kDim * kDim / 4; e += blockDim.x) {
      const float4 x = m4[e];
      nonzero |= (x.x != 0.f) | (x.y != 0.f) | (x.z != 0.f) | (x.w != 0.f);
    }
    if (!__syncthreads_or(nonzero)) {
      start = j;
      break;
    }
  }
  {
    const float4* b0 = reinterpret_cast<const float4*>(pairs + ((2LL * start + 1) * blocks) * block + base);
    float4* dst = reinterpret_cast<float4*>(state);
    for (int e = threadIdx.x; e < kDim * kDim / 4; e += blockDim.x) dst[e] = b0[e];
  }
  for (int j = start + 1; j < n; ++j) {
    __syncthreads();                 // the state written by the previous step is visible to the whole CTA
    affine_step(pairs + (2LL * j * blocks) * block + base, pairs + ((2LL * j + 1) * blocks) * block + base, state, state,
                tile_m, tile_s);
  }
  if (outgoing) {
    __syncthreads();
    affine_step(my_m + base, my_b + base, state, outgoing + base, tile_m, tile_s);
  }
}

}  // namespace
}  // namespace gdn_sm100

using namespace gdn_sm100;

extern "C" int actlize_la_sm100_abi_version(void) { return ACTLIZE_LA_SM100_ABI_VERSION; }
extern "C" int actlize_la_sm100_target_arch(void) { return 100; }
extern "C" const char* actlize_la_sm100_numerical_contract(void) {
  return "wy-splitbf16-state-bf16-out-sm100-v1";
}

namespace gdn_sm100 {
namespace {
// Host-visible failure record, one page of this library's own static storage per device, pinned and mapped by
// configure() (cudaHostRegister: nothing is allocated).  A kernel that gives up a bounded wait writes
// (code, block, site, chunk) here as well as into its device word, so the host can notice without synchronising.
constexpr int kMaxStatusDevices = 64;
alignas(4096) int g_status_pages[kMaxStatusDevices][1024];
bool g_status_mapped[kMaxStatusDevices] = {};

int map_status_page() {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return int(e);
  if (device < 0 || device >= kMaxStatusDevices) return int(cudaErrorInvalidDevice);
  if (g_status_mapped[device]) return 0;
  e = cudaHostRegister(g_status_pages[device], sizeof(g_status_pages[device]),
                       cudaHostRegisterMapped | cudaHostRegisterPortable);
  if (e != cudaSuccess) return int(e);
  int* on_device = nullptr;
  if ((e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&on_device), g_status_pages[device], 0)) != cudaSuccess)
    return int(e);
  if (int rc = set_status_mirror_umma(on_device)) return rc;
  if (int rc = set_status_mirror_gemm(on_device)) return rc;
  g_status_mapped[device] = true;
  return 0;
}
volatile int* status_page_of_current_device() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxStatusDevices || !g_status_mapped[device])
    return nullptr;
  return g_status_pages[device];
}
}  // namespace
}  // namespace gdn_sm100

extern "C" int actlize_la_sm100_configure(void) {
  if (int rc = configure_simt()) return rc;
  if (int rc = configure_umma()) return rc;
  if (int rc = configure_out_proj()) return rc;
  if (int rc = map_status_page()) return rc;
  return create_segment_streams();
}

extern "C" int actlize_la_sm100_select(int b, int t, int hk, int hv, int gate_fp32) {
  (void)gate_fp32;
  if (!geometry_ok(b, t, hk, hv)) return -1;
  for (const PolicyRow& row : kPolicyRows)
    if (row.b == b && row.t == t && row.hk == hk && row.hv == hv)
      return row.config | (row.segments << kSegmentShift) | (row.parallel << kParallelShift);
  // no measured row: integer rules (sm100_policy.py::default_parallel / default_segments are the same).  Parallel
  // sub-segments: as many as fill the 148 SMs with one walk CTA each, at least 8 chunks per sub-segment, at most 8.
  // Sequence segments (prepare of a later segment next to the walk of an earlier one) only pay while the walk
  // leaves SMs idle, i.e. when the walk is not split.
  const long long heads = (long long)b * hv, chunks = (t + kChunk - 1) / kChunk;
  long long parallel = 148 / heads;
  if (parallel > chunks / 8) parallel = chunks / 8;
  if (parallel > kMaxParallel) parallel = kMaxParallel;
  if (parallel < 1) parallel = 1;
  int segments = 1;
  if (heads <= 64 && parallel == 1) {
    int root = 0;
    while ((long long)(root + 1) * (root + 1) <= chunks / 8) ++root;
    segments = root < 1 ? 1 : (root > 8 ? 8 : root);
  }
  return kPolicyDefault | (kPolicyDefault == 1 ? (segments << kSegmentShift) | (int(parallel) << kParallelShift) : 0);
}

extern "C" long long actlize_la_sm100_workspace_bytes(int b, int t, int hk, int hv, int config) {
  if (!geometry_ok(b, t, hk, hv) || !config_ok(config)) return -1;
  const Geometry geo{b, t, hk, hv};
  return workspace_bytes(geo, segments_of(config, geo));
}

extern "C" int actlize_la_sm100_launches_per_forward(int config) {
  if (!config_ok(config)) return -1;
  if (config & kStageMask) return 1;
  const int segments = (config >> kSegmentShift) & 0xff;
  return ((config & 0xf) == 1 && segments > 1) ? 2 * segments : 2;
}

extern "C" int actlize_la_sm100_selftest_wait_timeout(int tag, void* stream) {
  return launch_wait_timeout_selftest(tag, static_cast<cudaStream_t>(stream));
}

extern "C" int actlize_la_sm100_device_status(int* status4, int reset) {
  if (!status4) return int(cudaErrorInvalidValue);
  volatile int* page = status_page_of_current_device();
  if (!page) return read_device_status(status4, reset);        // configure() has not run on this device
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return int(e);
  for (int i = 0; i < 4; ++i) status4[i] = page[i];
  if (reset) {
    for (int i = 0; i < 4; ++i) page[i] = 0;
    if (int rc = clear_device_status_umma()) return rc;
    if (int rc = clear_device_status_gemm()) return rc;
  }
  return 0;
}

extern "C" int actlize_la_sm100_last_failure(int* status4) {
  if (!status4) return int(cudaErrorInvalidValue);
  volatile int* page = status_page_of_current_device();
  for (int i = 0; i < 4; ++i) status4[i] = page ? page[i] : 0;
  return 0;
}

extern "C" int actlize_la_sm100_selftest_walk_stall(
    const void* q, const void* k, const void* v, const void* g, const void* beta, void* output,
    void* workspace, long long workspace_bytes_given, int b, int t, int hk, int hv, int gate_fp32, void* stream) {
  if (!q || !k || !v || !g || !beta || !output || !workspace) return int(cudaErrorInvalidValue);
  if (!geometry_ok(b, t, hk, hv) || t <= kChunk) return int(cudaErrorInvalidValue);     // at least two chunks
  const Geometry geo{b, t, hk, hv};
  if (workspace_bytes_given < workspace_bytes(geo) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return int(cudaErrorInvalidValue);
  const Inputs in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                  static_cast<const __nv_bfloat16*>(v), g, static_cast<const __nv_bfloat16*>(beta),
                  nullptr, static_cast<__nv_bfloat16*>(output), nullptr, gate_fp32 ? 1 : 0};
  return launch_walk_stall_selftest(in, geo, carve_workspace(workspace, geo), static_cast<cudaStream_t>(stream));
}

extern "C" int actlize_la_sm100_walk_plan_counts(int* counts2, int reset) {
  if (!counts2) return int(cudaErrorInvalidValue);
  return read_walk_plan_counts(counts2, reset);
}

namespace {
int run_forward(const Inputs& in, Geometry geo, const Workspace& ws, int config, int segments, cudaStream_t stream);
}

extern "C" int actlize_la_sm100_forward_prepared(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial, void* output, float* final_state,
    void* workspace, long long workspace_bytes_given,
    int b, int t, int hk, int hv, int gate_fp32, int config, void* opaque_stream) {
  if (!q || !k || !v || !g || !beta || !output || !workspace) return int(cudaErrorInvalidValue);
  if (!geometry_ok(b, t, hk, hv) || !config_ok(config)) return int(cudaErrorInvalidValue);
  Geometry geo{b, t, hk, hv};
  const int segments = segments_of(config, geo);
  if (workspace_bytes_given < workspace_bytes(geo, segments)) return int(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(output) & 15))
    return int(cudaErrorInvalidValue);
  if (output == workspace || (void*)final_state == workspace || (void*)final_state == output)
    return int(cudaErrorInvalidValue);
  if ((config & kUntilDecayedBit) && final_state) return int(cudaErrorInvalidValue);   // a cut-short walk has no final state
  if ((config & (kOffsetTailBit | kPairBit)) && !final_state) return int(cudaErrorInvalidValue);   // these passes write nothing else
  const Inputs in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                  static_cast<const __nv_bfloat16*>(v), g, static_cast<const __nv_bfloat16*>(beta),
                  initial, static_cast<__nv_bfloat16*>(output), final_state, gate_fp32 ? 1 : 0,
                  ((config & kHomogeneousBit) ? kWalkHomogeneous : 0) | ((config & kUntilDecayedBit) ? kWalkUntilDecayed : 0) |
                      ((config & kOffsetTailBit) ? kWalkTail : 0) | ((config & kPairBit) ? kWalkPair : 0)};
  const Workspace ws = carve_workspace(workspace, geo);
  return run_forward(in, geo, ws, config, segments, static_cast<cudaStream_t>(opaque_stream));
}

namespace {
int run_forward(const Inputs& in, Geometry geo, const Workspace& ws, int config, int segments, cudaStream_t stream) {
  if (segments > 1) {
    // Three streams.  The caller's: the first segment's prepare, then its walk, which so follows without an event
    // hop and claims its SMs before the second prepare kernel fills the device.  A second one (normal priority): the
    // prepare kernels of the later segments, forked behind the first prepare.  A high-priority third: the later
    // walks, each behind the previous walk and its own segment's prepare; as a walk ends, the next takes over its
    // SMs ahead of pending prepare blocks.  The caller's stream finally waits for the last walk.
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return int(e);
    if (device < 0 || device >= 64 || !g_streams[device].prepare) return int(cudaErrorNotReady);   // configure() first
    SegmentStreams& ss = g_streams[device];
    const int chunks = geo.chunks();
    for (int i = 0; i < segments; ++i) {
      geo.chunk_begin = int((long long)chunks * i / segments);
      geo.chunk_count = int((long long)chunks * (i + 1) / segments) - geo.chunk_begin;
      geo.parallel = parallel_of(config, geo.chunk_count);
      if (i == 0) {
        if (int rc = launch_prepare_tc(config, in, geo, ws, stream)) return rc;
        if ((e = cudaEventRecord(ss.start, stream)) != cudaSuccess) return int(e);
        if ((e = cudaStreamWaitEvent(ss.prepare, ss.start, 0)) != cudaSuccess) return int(e);
        if (int rc = launch_walk_tc(config, in, geo, ws, stream)) return rc;
        if ((e = cudaEventRecord(ss.walked[0], stream)) != cudaSuccess) return int(e);
        if ((e = cudaStreamWaitEvent(ss.walk, ss.walked[0], 0)) != cudaSuccess) return int(e);
      } else {
        if (int rc = launch_prepare_tc(config, in, geo, ws, ss.prepare)) return rc;
        if ((e = cudaEventRecord(ss.prepared[i], ss.prepare)) != cudaSuccess) return int(e);
        if ((e = cudaStreamWaitEvent(ss.walk, ss.prepared[i], 0)) != cudaSuccess) return int(e);
        if (int rc = launch_walk_tc(config, in, geo, ws, ss.walk)) return rc;
      }
    }
    if ((e = cudaEventRecord(ss.done, ss.walk)) != cudaSuccess) return int(e);
    return int(cudaStreamWaitEvent(stream, ss.done, 0));
  }
  geo.parallel = parallel_of(config, geo.segment_chunks());
  if (!(config & kWalkOnly)) {
    if (int rc = in.mixed                  ? launch_prepare_fused(in, geo, ws, stream)
                 : prepare_is_umma(config) ? launch_prepare_umma(in, geo, ws, stream)
                                           : launch_prepare_simt(in, geo, ws, stream))
      return rc;
  }
  if (config & kPrepareOnly) return 0;
  return walk_is_umma(config) ? launch_walk_umma(in, geo, ws, stream) : launch_walk_simt(in, geo, ws, stream);
}
}  // namespace

// --------------------------------------------------------------- forward on raw projection outputs
extern "C" long long actlize_la_sm100_projections_workspace_bytes(int b, int t, int hk, int hv, int config) {
  if (!geometry_ok(b, t, hk, hv) || !config_ok(config) || (config & 0xf) != 1 || (config & (kStageMask | kWalkFlagMask)))
    return -1;
  const Geometry geo{b, t, hk, hv};
  // the ordinary workspace plus the normalised keys and queries, each [B][T][Hk][128] BF16
  return ((workspace_bytes(geo, segments_of(config, geo)) + 255) & ~255LL) + 2 * (((long long)b * t * hk * kDim * 2 + 255) & ~255LL);
}

extern "C" int actlize_la_sm100_forward_projections(
    const void* mixed, long long mixed_row_stride, const void* a, const void* b_act, const float* a_log,
    const float* dt_bias, const float* initial, void* output, float* final_state,
    void* workspace, long long workspace_bytes_given,
    int b, int t, int hk, int hv, int config, void* opaque_stream) {
  if (!mixed || !a || !b_act || !a_log || !dt_bias || !output || !workspace) return int(cudaErrorInvalidValue);
  const long long need = actlize_la_sm100_projections_workspace_bytes(b, t, hk, hv, config);
  if (need < 0 || workspace_bytes_given < need) return int(cudaErrorInvalidValue);
  if (mixed_row_stride < (2LL * hk + hv) * kDim || (mixed_row_stride & 7) || (long long)b * t > INT_MAX ||
      (reinterpret_cast<uintptr_t>(mixed) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      (reinterpret_cast<uintptr_t>(output) & 15))
    return int(cudaErrorInvalidValue);
  Geometry geo{b, t, hk, hv};
  const int segments = segments_of(config, geo);
  const Workspace ws = carve_workspace(workspace, geo);
  Inputs in{};
  char* planes = static_cast<char*>(workspace) + ((workspace_bytes(geo, segments) + 255) & ~255LL);
  in.k_norm = reinterpret_cast<__nv_bfloat16*>(planes);
  in.q_norm = reinterpret_cast<__nv_bfloat16*>(planes + (((long long)b * t * hk * kDim * 2 + 255) & ~255LL));
  in.k = in.k_norm;                 // what the walk reads
  in.q = in.q_norm;
  in.initial = initial;
  in.output = static_cast<__nv_bfloat16*>(output);
  in.final_state = final_state;
  in.gate_fp32 = 1;
  in.mixed = static_cast<const __nv_bfloat16*>(mixed);
  in.mixed_stride = mixed_row_stride;
  in.act_a = static_cast<const __nv_bfloat16*>(a);
  in.act_b = static_cast<const __nv_bfloat16*>(b_act);
  in.a_log = a_log;
  in.dt_bias = dt_bias;
  return run_forward(in, geo, ws, config, segments, static_cast<cudaStream_t>(opaque_stream));
}

// ---------------------------------------------------------------------------------- packed sequences
namespace {
long long align256_ll(long long x) { return (x + 255) & ~255LL; }
long long varlen_table_bytes(int n_seqs) { return align256_ll(2LL * (n_seqs + 1) * (long long)sizeof(int)); }
}  // namespace

extern "C" long long actlize_la_sm100_varlen_workspace_bytes(long long total_tokens, int n_seqs, int hk, int hv) {
  if (total_tokens <= 0 || total_tokens > INT_MAX || n_seqs <= 0 || !geometry_ok(1, int(total_tokens), hk, hv)) return -1;
  // every sequence starts a new chunk, so each may add one partly filled chunk to ceil(total / 64)
  const long long max_chunks = (total_tokens + kChunk - 1) / kChunk + n_seqs;
  if (max_chunks * hv > INT_MAX / kDim || (long long)n_seqs * hv > INT_MAX / 8) return -1;
  return varlen_table_bytes(n_seqs) + max_chunks * hv * kBlockBytes;
}

extern "C" int actlize_la_sm100_forward_varlen(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial_states, void* output, float* final_states,
    void* workspace, long long workspace_bytes_given,
    const int* cu_seqlens_host, int n_seqs, int hk, int hv, int gate_fp32, void* opaque_stream) {
  if (!q || !k || !v || !g || !beta || !output || !workspace || !cu_seqlens_host) return int(cudaErrorInvalidValue);
  if (n_seqs <= 0 || cu_seqlens_host[0] != 0) return int(cudaErrorInvalidValue);
  for (int i = 0; i < n_seqs; ++i)
    if (cu_seqlens_host[i + 1] < cu_seqlens_host[i]) return int(cudaErrorInvalidValue);
  const int total = cu_seqlens_host[n_seqs];
  const long long need = actlize_la_sm100_varlen_workspace_bytes(total, n_seqs, hk, hv);
  if (need < 0 || workspace_bytes_given < need) return int(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(output) & 15))
    return int(cudaErrorInvalidValue);
  // offsets table: cu_seqlens[0..n] then chunk_prefix[0..n]
  std::vector<int> table(2 * (n_seqs + 1));
  int chunks = 0;
  for (int i = 0; i <= n_seqs; ++i) {
    table[i] = cu_seqlens_host[i];
    table[n_seqs + 1 + i] = chunks;
    if (i < n_seqs) chunks += (cu_seqlens_host[i + 1] - cu_seqlens_host[i] + kChunk - 1) / kChunk;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(opaque_stream);
  // pageable source: the runtime has staged the bytes when the call returns, so `table` may go out of scope
  cudaError_t e = cudaMemcpyAsync(workspace, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return int(e);
  Geometry geo{n_seqs, total, hk, hv};
  geo.varlen = static_cast<const int*>(workspace);
  geo.total_chunks = chunks;
  const Inputs in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                  static_cast<const __nv_bfloat16*>(v), g, static_cast<const __nv_bfloat16*>(beta),
                  initial_states, static_cast<__nv_bfloat16*>(output), final_states, gate_fp32 ? 1 : 0};
  const Workspace ws = carve_workspace(static_cast<char*>(workspace) + varlen_table_bytes(n_seqs), geo);
  if (int rc = launch_prepare_umma(in, geo, ws, stream)) return rc;
  return launch_walk_umma(in, geo, ws, stream);
}

extern "C" int actlize_la_sm100_forward_varlen_device(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial_states, void* output, float* final_states,
    void* workspace, long long workspace_bytes_given,
    const int* cu_seqlens_device, int n_seqs, long long total_tokens, int hk, int hv, int gate_fp32,
    void* opaque_stream) {
  if (!q || !k || !v || !g || !beta || !output || !workspace || !cu_seqlens_device) return int(cudaErrorInvalidValue);
  const long long need = actlize_la_sm100_varlen_workspace_bytes(total_tokens, n_seqs, hk, hv);
  if (need < 0 || workspace_bytes_given < need) return int(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(output) & 15))
    return int(cudaErrorInvalidValue);
  cudaStream_t stream = static_cast<cudaStream_t>(opaque_stream);
  varlen_table_kernel<<<1, 32, 0, stream>>>(cu_seqlens_device, n_seqs, int(total_tokens), static_cast<int*>(workspace));
  if (cudaError_t e = cudaGetLastError()) return int(e);
  Geometry geo{n_seqs, int(total_tokens), hk, hv};
  geo.varlen = static_cast<const int*>(workspace);
  // the host does not know the lengths: the grids and the workspace indexing use the upper bound (every sequence
  // may add one partly filled chunk); prepare blocks behind the real chunk count leave at once
  geo.total_chunks = int((total_tokens + kChunk - 1) / kChunk + n_seqs);
  const Inputs in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                  static_cast<const __nv_bfloat16*>(v), g, static_cast<const __nv_bfloat16*>(beta),
                  initial_states, static_cast<__nv_bfloat16*>(output), final_states, gate_fp32 ? 1 : 0};
  const Workspace ws = carve_workspace(static_cast<char*>(workspace) + varlen_table_bytes(n_seqs), geo);
  if (int rc = launch_prepare_umma(in, geo, ws, stream)) return rc;
  return launch_walk_umma(in, geo, ws, stream);
}

namespace {
// Segment boundaries of the host-buffer entry.  The transfers bound that path; what cannot overlap them is the last
// segment's compute and copy-out, so the segments taper towards the end (cumulative fraction 1 - (1 - i/n)^2:
// 44 %, 31 %, 19 %, 6 % for four) instead of being equal.  Every segment keeps at least one chunk.
int tapered_begin(int chunks, int i, int segments) {
  if (i >= segments) return chunks;
  const double rest = 1.0 - double(i) / segments;
  int begin = int(chunks * (1.0 - rest * rest) + 0.5);
  if (begin < i) begin = i;
  if (begin > chunks - (segments - i)) begin = chunks - (segments - i);
  return begin;
}

// Sequence segments of the host-buffer entry: the configuration's own count when it has one; otherwise the entry
// picks a pipeline depth itself, because its segments exist to overlap the PCIe transfers with the computation,
// whatever the device-resident forward prefers (tcgen05 family only: the other kernels cannot start mid-sequence).
int host_segments_of(int config, const Geometry& geo) {
  const int segments = segments_of(config, geo);
  if (segments > 1 || (config & 0xf) != 1 || (config & (kStageMask | kWalkFlagMask))) return segments;
  const int chunks = geo.chunks();
  return chunks >= 32 ? 4 : (chunks >= 8 ? 2 : 1);
}

struct Arena {
  long long q, k, v, g, beta, initial, output, final_state, workspace, total;
};
long long align256(long long x) { return (x + 255) & ~255LL; }
Arena arena_layout(int b, int t, int hk, int hv, int gate_fp32, int has_initial, int has_final, int config) {
  Arena a{};
  long long off = 0;
  auto take = [&](long long bytes) { long long at = off; off = align256(off + bytes); return at; };
  const long long qk = (long long)b * t * hk * kDim * 2, vv = (long long)b * t * hv * kDim * 2;
  const long long sc = (long long)b * t * hv, st = (long long)b * hv * kDim * kDim * 4;
  a.q = take(qk); a.k = take(qk); a.v = take(vv);
  a.g = take(sc * (gate_fp32 ? 4 : 2)); a.beta = take(sc * 2);
  a.initial = has_initial ? take(st) : -1;
  a.output = take(vv);
  a.final_state = has_final ? take(st) : -1;
  const Geometry geo{b, t, hk, hv};
  a.workspace = take(workspace_bytes(geo, host_segments_of(config, geo)));
  a.total = off;
  return a;
}
}  // namespace

extern "C" long long actlize_la_sm100_host_arena_bytes(int b, int t, int hk, int hv, int gate_fp32,
                                                       int has_initial, int has_final, int config) {
  if (!geometry_ok(b, t, hk, hv) || !config_ok(config)) return -1;
  return arena_layout(b, t, hk, hv, gate_fp32, has_initial, has_final, config).total;
}

extern "C" int actlize_la_sm100_forward_host(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial, void* output, float* final_state,
    void* device_arena, long long device_arena_bytes,
    int b, int t, int hk, int hv, int gate_fp32, int config, void* opaque_stream) {
  if (!q || !k || !v || !g || !beta || !output || !device_arena) return int(cudaErrorInvalidValue);
  if (!geometry_ok(b, t, hk, hv) || !config_ok(config)) return int(cudaErrorInvalidValue);
  if (reinterpret_cast<uintptr_t>(device_arena) & 255) return int(cudaErrorInvalidValue);
  const Arena a = arena_layout(b, t, hk, hv, gate_fp32, initial != nullptr, final_state != nullptr, config);
  if (device_arena_bytes < a.total) return int(cudaErrorInvalidValue);
  char* base = static_cast<char*>(device_arena);
  cudaStream_t stream = static_cast<cudaStream_t>(opaque_stream);
  const long long qk = (long long)b * t * hk * kDim * 2, vv = (long long)b * t * hv * kDim * 2;
  const long long sc = (long long)b * t * hv, st = (long long)b * hv * kDim * kDim * 4;
  cudaError_t e;
  {
    Geometry geo{b, t, hk, hv};
    const int segments = host_segments_of(config, geo);
    if (segments > 1) {
      // Pipelined form: the sequence is cut into the same chunk-aligned segments as the computation.
      // Inputs of segment i+1 travel host -> device on one copy stream while segment i is prepared and
      // walked, and finished output rows travel device -> host on another, so both PCIe directions and
      // the SMs are busy at the same time.
      int device = -1;
      if ((e = cudaGetDevice(&device)) != cudaSuccess) return int(e);
      if (device < 0 || device >= 64 || !g_streams[device].walk) return int(cudaErrorNotReady);   // configure() first
      SegmentStreams& ss = g_streams[device];
      const Inputs in{reinterpret_cast<const __nv_bfloat16*>(base + a.q), reinterpret_cast<const __nv_bfloat16*>(base + a.k),
                      reinterpret_cast<const __nv_bfloat16*>(base + a.v), base + a.g,
                      reinterpret_cast<const __nv_bfloat16*>(base + a.beta),
                      initial ? reinterpret_cast<const float*>(base + a.initial) : nullptr,
                      reinterpret_cast<__nv_bfloat16*>(base + a.output),
                      final_state ? reinterpret_cast<float*>(base + a.final_state) : nullptr, gate_fp32 ? 1 : 0};
      const Workspace ws = carve_workspace(base + a.workspace, geo);
      const int chunks = geo.chunks();
      const long long gate_bytes = gate_fp32 ? 4 : 2;
      if ((e = cudaEventRecord(ss.start, stream)) != cudaSuccess) return int(e);
      if ((e = cudaStreamWaitEvent(ss.copy_in, ss.start, 0)) != cudaSuccess) return int(e);
      if ((e = cudaStreamWaitEvent(ss.copy_out, ss.start, 0)) != cudaSuccess) return int(e);
      if (initial && (e = cudaMemcpyAsync(base + a.initial, initial, st, cudaMemcpyHostToDevice, ss.copy_in)) != cudaSuccess)
        return int(e);
      // gate and beta are small (6 bytes per token and value head): they travel whole, ahead of everything else,
      // instead of as two more short copies per segment
      if ((e = cudaMemcpyAsync(base + a.g, g, sc * gate_bytes, cudaMemcpyHostToDevice, ss.copy_in)) != cudaSuccess)
        return int(e);
      if ((e = cudaMemcpyAsync(base + a.beta, beta, sc * 2, cudaMemcpyHostToDevice, ss.copy_in)) != cudaSuccess)
        return int(e);
      for (int i = 0; i < segments; ++i) {
        geo.chunk_begin = tapered_begin(chunks, i, segments);
        geo.chunk_count = tapered_begin(chunks, i + 1, segments) - geo.chunk_begin;
        // one CTA per (batch, value head): the walks hide behind the transfers anyway, and the extra chunks that
        // parallel sub-segments walk only take memory bandwidth from the copies (measured 1.5 % slower with them)
        geo.parallel = 1;
        const long long t0 = (long long)geo.chunk_begin * kChunk;
        const long long rows = ((long long)(geo.chunk_begin + geo.chunk_count) * kChunk < t ?
                                (long long)(geo.chunk_begin + geo.chunk_count) * kChunk : t) - t0;
        for (int bb = 0; bb < b; ++bb) {      // a segment is contiguous within one batch element
          const long long tok = (long long)bb * t + t0;
          struct { long long dst; const void* src; long long row; } parts[3] = {
              {a.q, q, hk * kDim * 2LL}, {a.k, k, hk * kDim * 2LL}, {a.v, v, hv * kDim * 2LL}};
          for (auto& part : parts)
            if ((e = cudaMemcpyAsync(base + part.dst + tok * part.row, static_cast<const char*>(part.src) + tok * part.row,
                                     rows * part.row, cudaMemcpyHostToDevice, ss.copy_in)) != cudaSuccess)
              return int(e);
        }
        if ((e = cudaEventRecord(ss.arrived[i], ss.copy_in)) != cudaSuccess) return int(e);
        if ((e = cudaStreamWaitEvent(stream, ss.arrived[i], 0)) != cudaSuccess) return int(e);
        if (int rc = launch_prepare_tc(config, in, geo, ws, stream)) return rc;
        if ((e = cudaEventRecord(ss.prepared[i], stream)) != cudaSuccess) return int(e);
        if ((e = cudaStreamWaitEvent(ss.walk, ss.prepared[i], 0)) != cudaSuccess) return int(e);
        if (int rc = launch_walk_tc(config, in, geo, ws, ss.walk)) return rc;
        if ((e = cudaEventRecord(ss.walked[i], ss.walk)) != cudaSuccess) return int(e);
        if ((e = cudaStreamWaitEvent(ss.copy_out, ss.walked[i], 0)) != cudaSuccess) return int(e);
        for (int bb = 0; bb < b; ++bb) {
          const long long off = ((long long)bb * t + t0) * hv * kDim * 2;
          if ((e = cudaMemcpyAsync(static_cast<char*>(output) + off, base + a.output + off, rows * hv * kDim * 2,
                                   cudaMemcpyDeviceToHost, ss.copy_out)) != cudaSuccess)
            return int(e);
        }
      }
      if (final_state &&
          (e = cudaMemcpyAsync(final_state, base + a.final_state, st, cudaMemcpyDeviceToHost, ss.copy_out)) != cudaSuccess)
        return int(e);
      if ((e = cudaEventRecord(ss.copied, ss.copy_out)) != cudaSuccess) return int(e);
      if ((e = cudaStreamWaitEvent(stream, ss.copied, 0)) != cudaSuccess) return int(e);
      return int(cudaStreamSynchronize(stream));
    }
  }
#define GDN_COPY(dst, src, bytes, kind) \
  if ((e = cudaMemcpyAsync(dst, src, bytes, kind, stream)) != cudaSuccess) return int(e)
  GDN_COPY(base + a.q, q, qk, cudaMemcpyHostToDevice);
  GDN_COPY(base + a.k, k, qk, cudaMemcpyHostToDevice);
  GDN_COPY(base + a.v, v, vv, cudaMemcpyHostToDevice);
  GDN_COPY(base + a.g, g, sc * (gate_fp32 ? 4 : 2), cudaMemcpyHostToDevice);
  GDN_COPY(base + a.beta, beta, sc * 2, cudaMemcpyHostToDevice);
  if (initial) GDN_COPY(base + a.initial, initial, st, cudaMemcpyHostToDevice);
  const int rc = actlize_la_sm100_forward_prepared(
      base + a.q, base + a.k, base + a.v, base + a.g, base + a.beta,
      initial ? reinterpret_cast<const float*>(base + a.initial) : nullptr, base + a.output,
      final_state ? reinterpret_cast<float*>(base + a.final_state) : nullptr,
      base + a.workspace, a.total - a.workspace, b, t, hk, hv, gate_fp32, config, opaque_stream);
  if (rc) return rc;
  GDN_COPY(output, base + a.output, vv, cudaMemcpyDeviceToHost);
  if (final_state) GDN_COPY(final_state, base + a.final_state, st, cudaMemcpyDeviceToHost);
#undef GDN_COPY
  return int(cudaStreamSynchronize(stream));
}

extern "C" int actlize_la_sm100_fold_transitions(const float* pairs, int n_pairs, const float* my_transition,
                                                 const float* my_offset, float* incoming, float* outgoing,
                                                 int blocks, void* opaque_stream) {
  if (!pairs || !incoming || n_pairs <= 0 || blocks <= 0) return int(cudaErrorInvalidValue);
  if (outgoing && (!my_transition || !my_offset || outgoing == incoming)) return int(cudaErrorInvalidValue);
  fold_transitions_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(opaque_stream)>>>(
      pairs, n_pairs, blocks, incoming, outgoing, my_transition, my_offset);
  return int(cudaGetLastError());
}

extern "C" int actlize_la_sm100_apply_transition(const float* transition, const float* offset,
                                                 const float* state_in, float* state_out,
                                                 int blocks, void* opaque_stream) {
  if (!transition || !offset || !state_in || !state_out || blocks <= 0 || state_in == state_out)
    return int(cudaErrorInvalidValue);
  apply_transition_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(opaque_stream)>>>(
      transition, offset, state_in, state_out);
  return int(cudaGetLastError());
}
