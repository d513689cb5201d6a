// Memory-bound companions of the chunked forward: the step before it (Q/K normalisation and gate
// activation), the single-token decode step on the same state layout, and the gated RMSNorm after it.
// Each is one streaming kernel whose roofline is HBM bandwidth; none needs tensor cores.
//
// Reference behaviour restated here (paths relative to the reference tree):
//   prepare_inputs   csrc/serving/prefill.cu:45-70 and csrc/serving/runtime.cuh:48-52
//                    (q,k <- x * rsqrt(sum x^2 + 1e-6) per 128-vector, v copied,
//                     g = -exp(A_log) * softplus(a + dt_bias) with the z > 20 branch, beta = sigmoid(b))
//   decode_step      actlize_la/reference/gdn_chunk_ref.py:135-143 (token recurrence), kernel analogue
//                    csrc/serving/gdn.cu:152 (recurrent_gdn); state kept in the public K-by-V order
//   rmsnorm_gated    csrc/output_gate/output_gate.cu:4-5,73-92 (out = y * rsqrt(mean y^2 + 1e-6) * w * silu(z))
#include "actlize_la_sm100.h"
#include "gdn_common.cuh"

#include <climits>

namespace gdn_sm100 {
namespace {

__device__ __forceinline__ float lo_bf16(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float hi_bf16(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }

// 16 lanes per 128-wide head vector (8 BF16 = 16 bytes per lane); a 256-thread CTA covers 64 consecutive vectors in
// four sweeps of 16 and issues the loads of all sweeps first (four 16-byte loads in flight per thread).
constexpr int kPrepSweeps = 4;
__global__ void __launch_bounds__(256)
prepare_inputs_kernel(const __nv_bfloat16* __restrict__ mixed, long long mixed_stride,
                      const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                      const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                      __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
                      float* __restrict__ g, __nv_bfloat16* __restrict__ beta, long long tokens, int hk, int hv) {
  const int heads = 2 * hk + hv;
  const int lane = threadIdx.x & 15;
  const long long first = (long long)blockIdx.x * (16 * kPrepSweeps) + (threadIdx.x >> 4);
  const long long vectors = tokens * heads;
  uint4 xs[kPrepSweeps];
#pragma unroll
  for (int r = 0; r < kPrepSweeps; ++r) {
    const long long slot = first + r * 16;
    const long long vec = slot < vectors ? slot : vectors - 1;     // idle groups redo the last vector and store nothing
    xs[r] = *reinterpret_cast<const uint4*>(mixed + (vec / heads) * mixed_stride + (vec % heads) * kDim + lane * 8);
  }
#pragma unroll
  for (int r = 0; r < kPrepSweeps; ++r) {
    const long long slot = first + r * 16;
    const bool live = slot < vectors;
    const long long vec = live ? slot : vectors - 1;
    const long long token = vec / heads;
    const int h = int(vec % heads);
    const uint4 x = xs[r];
    if (h < 2 * hk) {
      float f[8] = {lo_bf16(x.x), hi_bf16(x.x), lo_bf16(x.y), hi_bf16(x.y),
                    lo_bf16(x.z), hi_bf16(x.z), lo_bf16(x.w), hi_bf16(x.w)};
      float square = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) square = fmaf(f[i], f[i], square);
#pragma unroll
      for (int d = 8; d; d >>= 1) square += __shfl_xor_sync(0xffffffffu, square, d, 16);
      const float factor = rsqrtf(square + 1e-6f);
      uint4 o;
      o.x = pack_bf16(f[0] * factor, f[1] * factor);
      o.y = pack_bf16(f[2] * factor, f[3] * factor);
      o.z = pack_bf16(f[4] * factor, f[5] * factor);
      o.w = pack_bf16(f[6] * factor, f[7] * factor);
      __nv_bfloat16* dst = (h < hk ? q : k) + (token * hk + (h % hk)) * kDim + lane * 8;
      if (live) *reinterpret_cast<uint4*>(dst) = o;
    } else {
      const int vh = h - 2 * hk;
      if (live) *reinterpret_cast<uint4*>(v + (token * hv + vh) * kDim + lane * 8) = x;
      if (live && lane == 0) {
        const long long at = token * hv + vh;
        const float z = __bfloat162float(a[at]) + dt_bias[vh];
        g[at] = -expf(a_log[vh]) * (z > 20.f ? z : log1pf(expf(z)));
        beta[at] = __float2bfloat16_rn(1.f / (1.f + expf(-__bfloat162float(b[at]))));
      }
    }
  }
}

// One CTA per (batch, value head), 256 threads: thread = (value column, half of the 128 key rows).  Its 64
// state entries live in registers, so the state is read once and written once (128 KiB of traffic per
// head and step); the two row halves meet through shared memory for k^T S and q^T S.
__global__ void __launch_bounds__(256)
decode_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const void* __restrict__ g,
                   const __nv_bfloat16* __restrict__ beta, float* __restrict__ state,
                   __nv_bfloat16* __restrict__ out, int hk, int hv, int gate_fp32) {
  __shared__ float sk[kDim], sq[kDim], partial[2][kDim];
  const int bh = blockIdx.x, col = threadIdx.x & (kDim - 1), half = threadIdx.x >> 7;
  const int bidx = bh / hv, vh = bh % hv;
  const long long qk_at = ((long long)bidx * hk + vh / (hv / hk)) * kDim;
  if (half == 0) sk[col] = __bfloat162float(k[qk_at + col]);
  else sq[col] = __bfloat162float(q[qk_at + col]);
  const float decay = expf(load_gate(g, bh, gate_fp32));
  const float bt = __bfloat162float(beta[bh]);
  const float value = __bfloat162float(v[(long long)bh * kDim + col]);
  float* column = state + ((long long)bh * kDim + half * 64) * kDim + col;
  float s[64];
#pragma unroll
  for (int r = 0; r < 64; ++r) s[r] = column[r * kDim] * decay;
  __syncthreads();
  const float* kk = sk + half * 64;
  const float* qq = sq + half * 64;
  float kv = 0.f;
#pragma unroll
  for (int r = 0; r < 64; ++r) kv = fmaf(kk[r], s[r], kv);
  partial[half][col] = kv;
  __syncthreads();
  const float delta = bt * (value - (partial[0][col] + partial[1][col]));
  float o = 0.f;
#pragma unroll
  for (int r = 0; r < 64; ++r) {
    s[r] = fmaf(kk[r], delta, s[r]);
    o = fmaf(qq[r], s[r], o);
    column[r * kDim] = s[r];
  }
  __syncthreads();
  partial[half][col] = o;
  __syncthreads();
  if (half == 0) out[(long long)bh * kDim + col] = __float2bfloat16_rn((partial[0][col] + partial[1][col]) * kScale);
}

// Verify step (speculative decoding): `width` draft tokens per request run through the same recurrence with the
// state held in registers and NOT written back; besides the outputs it records delta_t = beta_t (v_t - k_t^T S),
// from which commit_step_kernel later applies the accepted prefix.  Thread layout as in decode_step_kernel; the
// arithmetic per token is the decode step's, operation for operation.
__global__ void __launch_bounds__(256)
verify_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const void* __restrict__ g,
                   const __nv_bfloat16* __restrict__ beta, const float* __restrict__ state,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ delta_out, int width, int hk, int hv,
                   int gate_fp32) {
  __shared__ float sk[2][kDim], sq[2][kDim], partial[2][kDim];
  const int bh = blockIdx.x, col = threadIdx.x & (kDim - 1), half = threadIdx.x >> 7;
  const int bidx = bh / hv, vh = bh % hv, kh = vh / (hv / hk);
  const float* column = state + ((long long)bh * kDim + half * 64) * kDim + col;
  float s[64];
#pragma unroll
  for (int r = 0; r < 64; ++r) s[r] = column[r * kDim];
  for (int t = 0; t < width; ++t) {
    const long long token = (long long)bidx * width + t;
    const long long qk_at = (token * hk + kh) * kDim, head = token * hv + vh;
    float* skt = sk[t & 1];
    float* sqt = sq[t & 1];
    if (half == 0) skt[col] = __bfloat162float(k[qk_at + col]);
    else sqt[col] = __bfloat162float(q[qk_at + col]);
    const float decay = expf(load_gate(g, head, gate_fp32));
    const float bt = __bfloat162float(beta[head]);
    const float value = __bfloat162float(v[head * kDim + col]);
#pragma unroll
    for (int r = 0; r < 64; ++r) s[r] *= decay;
    __syncthreads();
    const float* kk = skt + half * 64;
    const float* qq = sqt + half * 64;
    float kv = 0.f;
#pragma unroll
    for (int r = 0; r < 64; ++r) kv = fmaf(kk[r], s[r], kv);
    partial[half][col] = kv;
    __syncthreads();
    const float delta = bt * (value - (partial[0][col] + partial[1][col]));
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < 64; ++r) {
      s[r] = fmaf(kk[r], delta, s[r]);
      o = fmaf(qq[r], s[r], o);
    }
    __syncthreads();
    partial[half][col] = o;
    __syncthreads();
    if (half == 0) {
      out[head * kDim + col] = __float2bfloat16_rn((partial[0][col] + partial[1][col]) * kScale);
      delta_out[head * kDim + col] = delta;
    }
    __syncthreads();      // `partial` is rewritten by the next token
  }
}

// Commit: apply the first counts[b] recorded updates, S <- e^{g_t} S + k_t delta_t^T, to the state in place.
__global__ void __launch_bounds__(256)
commit_step_kernel(const __nv_bfloat16* __restrict__ k, const void* __restrict__ g,
                   const float* __restrict__ delta, const int* __restrict__ counts, float* __restrict__ state,
                   int width, int hk, int hv, int gate_fp32) {
  __shared__ float sk[2][kDim];
  const int bh = blockIdx.x, col = threadIdx.x & (kDim - 1), half = threadIdx.x >> 7;
  const int bidx = bh / hv, vh = bh % hv, kh = vh / (hv / hk);
  const int count = min(max(counts[bidx], 0), width);
  if (count == 0) return;
  float* column = state + ((long long)bh * kDim + half * 64) * kDim + col;
  float s[64];
#pragma unroll
  for (int r = 0; r < 64; ++r) s[r] = column[r * kDim];
  for (int t = 0; t < count; ++t) {
    const long long token = (long long)bidx * width + t;
    const long long head = token * hv + vh;
    if (half == 0) sk[t & 1][col] = __bfloat162float(k[(token * hk + kh) * kDim + col]);
    const float decay = expf(load_gate(g, head, gate_fp32));
    const float d = delta[head * kDim + col];
    __syncthreads();
    const float* kk = sk[t & 1] + half * 64;
#pragma unroll
    for (int r = 0; r < 64; ++r) s[r] = fmaf(kk[r], d, s[r] * decay);
  }
#pragma unroll
  for (int r = 0; r < 64; ++r) column[r * kDim] = s[r];
}

// 16 lanes per 128-wide row (16 bytes per lane and tensor); a 256-thread CTA covers 64 consecutive rows in four
// sweeps of 16, and every thread issues the loads of all four sweeps before it touches the data, so that eight
// 16-byte loads per thread are in flight (one row per thread group at a time left the memory system idle).
constexpr int kNormSweeps = 4;
__global__ void __launch_bounds__(256)
rmsnorm_gated_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                     const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out, long long rows) {
  const int lane = threadIdx.x & 15;
  const long long first = (long long)blockIdx.x * (16 * kNormSweeps) + (threadIdx.x >> 4);
  uint4 yy[kNormSweeps], zz[kNormSweeps];
#pragma unroll
  for (int r = 0; r < kNormSweeps; ++r) {
    const long long slot = first + r * 16;
    const long long row = slot < rows ? slot : rows - 1;     // idle groups redo the last row and store nothing
    yy[r] = *reinterpret_cast<const uint4*>(y + row * kDim + lane * 8);
    zz[r] = *reinterpret_cast<const uint4*>(z + row * kDim + lane * 8);
  }
  const uint4 ww = *reinterpret_cast<const uint4*>(weight + lane * 8);
  const uint32_t wp[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
  for (int r = 0; r < kNormSweeps; ++r) {
    const long long slot = first + r * 16;
    const uint32_t yp[4] = {yy[r].x, yy[r].y, yy[r].z, yy[r].w}, zp[4] = {zz[r].x, zz[r].y, zz[r].z, zz[r].w};
    float yf[8], square = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      yf[2 * i] = lo_bf16(yp[i]);
      yf[2 * i + 1] = hi_bf16(yp[i]);
      square = fmaf(yf[2 * i], yf[2 * i], fmaf(yf[2 * i + 1], yf[2 * i + 1], square));
    }
#pragma unroll
    for (int d = 8; d; d >>= 1) square += __shfl_xor_sync(0xffffffffu, square, d, 16);
    const float rstd = rsqrtf(square * (1.f / kDim) + 1e-6f);
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float z0 = lo_bf16(zp[i]), z1 = hi_bf16(zp[i]);
      const float r0 = yf[2 * i] * rstd * lo_bf16(wp[i]) * (z0 / (1.f + expf(-z0)));
      const float r1 = yf[2 * i + 1] * rstd * hi_bf16(wp[i]) * (z1 / (1.f + expf(-z1)));
      packed[i] = pack_bf16(r0, r1);
    }
    if (slot < rows)
      *reinterpret_cast<uint4*>(out + slot * kDim + lane * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

}  // namespace
}  // namespace gdn_sm100

using namespace gdn_sm100;

extern "C" int actlize_la_sm100_prepare_inputs(
    const void* mixed, long long mixed_row_stride, const void* a, const void* b, const float* a_log,
    const float* dt_bias, void* q, void* k, void* v, float* g, void* beta, long long tokens, int hk, int hv,
    void* stream) {
  if (!mixed || !a || !b || !a_log || !dt_bias || !q || !k || !v || !g || !beta) return int(cudaErrorInvalidValue);
  if (tokens <= 0 || hk <= 0 || hv <= 0 || hv % hk || mixed_row_stride < (2LL * hk + hv) * kDim ||
      (mixed_row_stride & 7) || (reinterpret_cast<uintptr_t>(mixed) & 15))
    return int(cudaErrorInvalidValue);
  const long long vectors = tokens * (2LL * hk + hv);
  const long long ctas = (vectors + 16 * kPrepSweeps - 1) / (16 * kPrepSweeps);
  if (ctas > INT_MAX) return int(cudaErrorInvalidValue);
  prepare_inputs_kernel<<<(unsigned)ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(mixed), mixed_row_stride, static_cast<const __nv_bfloat16*>(a),
      static_cast<const __nv_bfloat16*>(b), a_log, dt_bias, static_cast<__nv_bfloat16*>(q),
      static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v), g, static_cast<__nv_bfloat16*>(beta), tokens, hk, hv);
  return int(cudaGetLastError());
}

extern "C" int actlize_la_sm100_decode_step(
    const void* q, const void* k, const void* v, const void* g, const void* beta, float* state, void* output,
    int batch, int hk, int hv, int gate_fp32, void* stream) {
  if (!q || !k || !v || !g || !beta || !state || !output) return int(cudaErrorInvalidValue);
  if (batch <= 0 || hk <= 0 || hv <= 0 || hv % hk || (long long)batch * hv > INT_MAX) return int(cudaErrorInvalidValue);
  decode_step_kernel<<<batch * hv, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      g, static_cast<const __nv_bfloat16*>(beta), state, static_cast<__nv_bfloat16*>(output), hk, hv, gate_fp32 ? 1 : 0);
  return int(cudaGetLastError());
}

extern "C" int actlize_la_sm100_verify_step(
    const void* q, const void* k, const void* v, const void* g, const void* beta, const float* state, void* output,
    float* delta, int batch, int width, int hk, int hv, int gate_fp32, void* stream) {
  if (!q || !k || !v || !g || !beta || !state || !output || !delta) return int(cudaErrorInvalidValue);
  if (batch <= 0 || width <= 0 || width > 64 || hk <= 0 || hv <= 0 || hv % hk || (long long)batch * hv > INT_MAX)
    return int(cudaErrorInvalidValue);
  verify_step_kernel<<<batch * hv, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      g, static_cast<const __nv_bfloat16*>(beta), state, static_cast<__nv_bfloat16*>(output), delta, width, hk, hv,
      gate_fp32 ? 1 : 0);
  return int(cudaGetLastError());
}

extern "C" int actlize_la_sm100_commit_step(const void* k, const void* g, const float* delta, const int* counts,
                                            float* state, int batch, int width, int hk, int hv, int gate_fp32,
                                            void* stream) {
  if (!k || !g || !delta || !counts || !state) return int(cudaErrorInvalidValue);
  if (batch <= 0 || width <= 0 || width > 64 || hk <= 0 || hv <= 0 || hv % hk || (long long)batch * hv > INT_MAX)
    return int(cudaErrorInvalidValue);
  commit_step_kernel<<<batch * hv, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k), g, delta, counts, state, width, hk, hv, gate_fp32 ? 1 : 0);
  return int(cudaGetLastError());
}

extern "C" int actlize_la_sm100_rmsnorm_gated(const void* y, const void* z, const void* weight, void* out,
                                              long long rows, void* stream) {
  if (!y || !z || !weight || !out || rows <= 0 || (rows + 63) / 64 > INT_MAX) return int(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return int(cudaErrorInvalidValue);
  rmsnorm_gated_kernel<<<(unsigned)((rows + 16 * kNormSweeps - 1) / (16 * kNormSweeps)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(z),
      static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), rows);
  return int(cudaGetLastError());
}
