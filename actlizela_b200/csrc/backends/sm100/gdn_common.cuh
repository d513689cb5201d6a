// Shared definitions of the sm_100a gated-delta-rule backend: geometry, the workspace
// layout handed from the prepare kernel to the chunk walk, and small device helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ != 1000)
#error "the cuda_sm100 backend is built for sm_100a only (nvcc -gencode arch=compute_100a,code=sm_100a)"
#endif

namespace gdn_sm100 {

constexpr int kChunk = 64;    // tokens per chunk
constexpr int kDim = 128;     // key and value head dimension
constexpr float kScale = 0.08838834764831845f;  // 1/sqrt(128), applied exactly once

struct Geometry {
  int batch, sequence, key_heads, value_heads;
  // A launch may cover a contiguous range of chunks only (sequence segment); 0 chunks = the whole sequence.
  int chunk_begin = 0, chunk_count = 0;
  // tcgen05 walk only: the launch's chunk range is cut into `parallel` sub-segments per (batch, value head), walked by
  // as many CTAs at the same time (0 or 1 = one CTA walks the whole range); see walk_umma_kernel.
  int parallel = 0;
  // Packed variable-length mode (tcgen05 kernels only): the tensors are [1, sequence = total tokens, H, ...],
  // `batch` is the number of sequences and `varlen` points at 2 (batch + 1) device integers: the token offsets
  // cu_seqlens[0..batch] followed by the chunk offsets chunk_prefix[0..batch] (every sequence starts a new chunk);
  // `total_chunks` = chunk_prefix[batch].  Workspace blocks are then indexed hv * total_chunks + global chunk.
  const int* varlen = nullptr;
  int total_chunks = 0;
  __host__ __device__ int chunks() const { return varlen ? total_chunks : (sequence + kChunk - 1) / kChunk; }
  __host__ __device__ int segment_chunks() const { return chunk_count ? chunk_count : chunks(); }
  __host__ __device__ bool first_segment() const { return chunk_begin == 0; }
  __host__ __device__ bool last_segment() const { return chunk_begin + segment_chunks() == chunks(); }
  __host__ __device__ int group() const { return value_heads / key_heads; }
  __host__ __device__ long long blocks() const {
    return varlen ? (long long)value_heads * total_chunks : (long long)batch * value_heads * chunks();
  }
};

// Parallel sub-segments of a walk over `chunks` chunks: sub-segment r covers [sub_segment_begin(r), sub_segment_begin(r + 1)).
// Every CTA but the last walks on into its successor's leading chunks (about kNominalReach of them at typical gates),
// so the last sub-segment is made that much longer than the others and all CTAs finish together; ranges too short
// for that are cut evenly.
constexpr int kNominalReach = 4;
__host__ __device__ inline int sub_segment_begin(int chunks, int r, int parallel) {
  if (r <= 0) return 0;
  if (r >= parallel) return chunks;
  const int body = chunks - kNominalReach;
  return int((long long)(body >= parallel * kNominalReach ? body : chunks) * r / parallel);
}

// Packed mode: the sequence that owns global chunk `gchunk` (largest s with chunk_prefix[s] <= gchunk; empty
// sequences share their successor's offset and are skipped by the search).
__device__ __forceinline__ int varlen_sequence_of(const int* chunk_prefix, int count, int gchunk) {
  int lo = 0, hi = count;          // invariant: chunk_prefix[lo] <= gchunk < chunk_prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_prefix[mid] <= gchunk) lo = mid; else hi = mid;
  }
  return lo;
}

// Workspace: structure-of-arrays planes, one entry per (batch, value head, chunk) block,
// block index = (b * Hv + hv) * chunks + c.  W is stored TRANSPOSED (key-dimension-major), the orientation the
// tensor-core kernels produce and consume it in: the prepare kernel's accumulator holds W^T with the key index on the
// tensor-memory lanes, and the walk reads W^T as an MN-major B operand.  U is token-major: the walk's chain warps
// read it one value per lane.  Per block:
//   w_hi, w_lo  BF16 [128][64]  W^T, W = T (beta K Gamma), split W ~= hi + lo        (key dim, token)
//   u           FP32 [64][128]  U = T (beta V)                                       (token, value dim)
//   p           BF16 [64][64]   tril(Q K^T * exp(prefix_i - prefix_j)) / sqrt(128)
//   gates       FP32 [192]      [0,64): exp(prefix_last - prefix_i), 0 for padding rows;
//                               [64]: exp(prefix_last); [65] (tcgen05 prepare only): non-zero when some token of the
//                               chunk is not a contraction of the state (beta < 0 or beta |k|^2 > 2);
//                               [128,192): exp(prefix_i) / sqrt(128), the scale the walk applies to the rows of its
//                               Q tile (the scaled queries are not stored: the walk reads q itself); rest unused
// plus, when the sequence is walked in segments, one FP32 [128][128] state per (batch, value head)
// that carries the state from one segment's walk to the next (K-by-V order, like the public state).
struct Workspace {
  __nv_bfloat16* w_hi;
  __nv_bfloat16* w_lo;
  float* u;
  __nv_bfloat16* p;
  float* gates;
  float* carry;
};
// element (token, dim) of a transposed [128][64] plane (w_hi, w_lo) of block `block`
__host__ __device__ inline long long transposed_index(long long block, int token, int dim) {
  return block * (kChunk * kDim) + (long long)dim * kChunk + token;
}

constexpr int kGateWords = 192, kGateQueryScale = 128;     // words per gate vector; first word of the query scales
constexpr long long kBlockBytes = 2LL * kChunk * kDim * 2 + kChunk * kDim * 4 + kChunk * kChunk * 2 + kGateWords * 4;

inline __host__ long long workspace_bytes(const Geometry& g, int segments = 1) {
  return g.blocks() * kBlockBytes + (segments > 1 ? (long long)g.batch * g.value_heads * kDim * kDim * 4 : 0);
}

// Carve the planes out of one caller-owned allocation (256-byte aligned base required).
inline __host__ Workspace carve_workspace(void* base, const Geometry& g) {
  char* p = static_cast<char*>(base);
  const long long n = g.blocks();
  Workspace w;
  w.w_hi = reinterpret_cast<__nv_bfloat16*>(p);  p += n * kChunk * kDim * 2;
  w.w_lo = reinterpret_cast<__nv_bfloat16*>(p);  p += n * kChunk * kDim * 2;
  w.u = reinterpret_cast<float*>(p);             p += n * kChunk * kDim * 4;
  w.p = reinterpret_cast<__nv_bfloat16*>(p);     p += n * kChunk * kChunk * 2;
  w.gates = reinterpret_cast<float*>(p);         p += n * kGateWords * 4;
  w.carry = reinterpret_cast<float*>(p);         // only backed by memory when segments > 1
  return w;
}

struct Inputs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const void* g;
  const __nv_bfloat16* beta;
  const float* initial;   // nullable
  __nv_bfloat16* output;
  float* final_state;     // nullable
  int gate_fp32;
  // tcgen05 walk only, for the sequence-parallel scheme:
  //   kWalkHomogeneous  treat U as zero (the state-transition pass: V = 0)
  //   kWalkUntilDecayed stop a (batch, value head) walk at the first chunk boundary where the decay accumulated
  //                     since the walk's start is below exp(-40); later outputs are left as they are
  //   kWalkTail         offset pass: from zero, only the suffix of the range that decides the outgoing state; no
  //                     output rows; final_state receives that state
  //   kWalkPair         kWalkTail and kWalkHomogeneous (from an identity state made in the kernel) in one launch,
  //                     two CTAs per (batch, value head); final_state is then [2][B][Hv][128][128] = (M, b)
  int walk_flags = 0;
  // Fused input preparation (tcgen05 prepare kernel only): q, k, v are then read from the packed projection
  // rows `mixed` [B*T][mixed_stride] = [q heads | k heads | v heads] x 128, normalised in shared memory; the gate and
  // beta come from the raw activations `act_a`, `act_b` [B*T][Hv] with the per-head constants `a_log`, `dt_bias`;
  // the normalised keys are written to `k_norm` [B][T][Hk][128] for the walk (which gets it as its `k`).
  const __nv_bfloat16* mixed = nullptr;
  long long mixed_stride = 0;
  const __nv_bfloat16* act_a = nullptr;
  const __nv_bfloat16* act_b = nullptr;
  const float* a_log = nullptr;
  const float* dt_bias = nullptr;
  __nv_bfloat16* k_norm = nullptr;
  __nv_bfloat16* q_norm = nullptr;      // likewise the normalised queries [B][T][Hk][128] (the walk gets it as its `q`)
};
constexpr int kWalkHomogeneous = 1, kWalkUntilDecayed = 2;
constexpr int kWalkTail = 8;              // offset pass: walk, from zero, only the suffix that decides the outgoing state
constexpr int kWalkPair = 16;             // offset pass and transition pass in one launch, two CTAs per (batch, value head);
                                          // final_state then is the block [2][B][Hv][128][128] = (transitions, offsets)
constexpr int kWalkSelftestStall = 4;     // the TMA producer stops after the first chunk (failure-detection self-test)
constexpr float kDecayedLog2 = -40.f * 1.4426950408889634f;

__device__ __forceinline__ float load_gate(const void* g, long long index, int gate_fp32) {
  return gate_fp32 ? static_cast<const float*>(g)[index]
                   : __bfloat162float(static_cast<const __nv_bfloat16*>(g)[index]);
}

// x ~= hi + lo with both parts BF16 (16 significant bits in total).
__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo_elem, hi_elem);   // .x = first (low half)
  return *reinterpret_cast<uint32_t*>(&v);
}

// Inclusive prefix sum of 64 gate values held one per thread by two warps (threads 0..63).
// `carry` is a shared float used to pass the first warp's total to the second.
__device__ __forceinline__ float chunk_prefix64(float x, int tid, float* carry) {
  const int lane = tid & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    float y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  if (tid == 31) *carry = x;
  __syncthreads();
  if (tid >= 32 && tid < 64) x += *carry;
  return x;
}

// Launchers implemented by the kernel translation units; each returns a cudaError_t value.
int launch_prepare_simt(const Inputs&, const Geometry&, const Workspace&, cudaStream_t);
int launch_walk_simt(const Inputs&, const Geometry&, const Workspace&, cudaStream_t);
int configure_simt();
int launch_prepare_umma(const Inputs&, const Geometry&, const Workspace&, cudaStream_t);
int launch_prepare_fused(const Inputs&, const Geometry&, const Workspace&, cudaStream_t);   // Inputs::mixed etc. set
int launch_walk_umma(const Inputs&, const Geometry&, const Workspace&, cudaStream_t);
int configure_umma();
int read_device_status(int* host_out4, int reset);
int read_walk_plan_counts(int* host_out2, int reset);
int launch_wait_timeout_selftest(int tag, cudaStream_t);
int launch_walk_stall_selftest(const Inputs&, const Geometry&, const Workspace&, cudaStream_t);
// host-visible failure record and poll limit, per translation unit that holds tensor-core kernels
int set_status_mirror_umma(int* device_pointer);
int clear_device_status_umma();
int set_status_mirror_gemm(int* device_pointer);
int clear_device_status_gemm();
// out_proj GEMM of the step after the path (out_proj.cu)
int configure_out_proj();

}  // namespace gdn_sm100
