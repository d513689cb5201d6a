// FP32 CUDA-core implementation of the two stages (configuration "simt").
//
// It exists as an independent device-side cross-check of the tensor-core kernels: the same
// workspace layout is produced and consumed, so either stage can be exchanged with its
// tcgen05 counterpart when a numerical difference has to be located.  All contractions are
// plain FP32 FMAs; only the quantities the tensor-core path rounds to BF16 (P, scaled Q) or to a
// BF16 hi+lo pair (W) are rounded.
//
// Math (per 64-token chunk, value head h, key head h / (Hv/Hk)); p = inclusive prefix of g:
//   A = tril(beta_i (k_i.k_j) exp(p_i-p_j), -1),  T = (I+A)^-1
//   W = T diag(beta exp(p)) K,  U = T diag(beta) V,  P = tril((q_i.k_j) exp(p_i-p_j)) / sqrt(128)
//   N = U - W S,  O = (Q exp(p)/sqrt(128)) S + P N,  S <- exp(p_last) S + K^T (N * exp(p_last-p))
// which is the reference's WY chunk form (tests/wy_cpu.py:44-88; kernels
// csrc/gdn_chunk/gdn_wy_ppu.cu:7-292 prepare/state/output).
#include "gdn_common.cuh"

namespace gdn_sm100 {
namespace {

constexpr int kPad = kDim + 1;
constexpr int kPrepareThreads = 256;
constexpr int kPrepareSmem = (2 * kChunk * kPad + kChunk * (kChunk + 1) + 4 * kChunk + 8) * 4;

__global__ void __launch_bounds__(kPrepareThreads)
prepare_simt_kernel(Inputs in, Geometry geo, Workspace ws) {
  extern __shared__ float smem[];
  float* sK = smem;                         // [64][129]
  float* sX = sK + kChunk * kPad;           // [64][129]  Q, later V
  float* sT = sX + kChunk * kPad;           // [64][65]   A, then T in place
  float* sp = sT + kChunk * (kChunk + 1);   // [64] prefix
  float* sbeta = sp + kChunk;               // [64]
  float* scoef = sbeta + kChunk;            // [64] beta * exp(p)
  float* sexp = scoef + kChunk;             // [64] exp(p)
  float* carry = sexp + kChunk;

  const int tid = threadIdx.x;
  const int chunk = blockIdx.x % geo.chunks();
  const int bh = blockIdx.x / geo.chunks();
  const int b = bh / geo.value_heads, hv = bh % geo.value_heads;
  const int hk = hv / geo.group();
  const int t0 = chunk * kChunk;
  const int valid = min(kChunk, geo.sequence - t0);
  const long long block = (long long)bh * geo.chunks() + chunk;

  float gate = 0.f, beta = 0.f;
  if (tid < valid) {
    const long long gi = ((long long)b * geo.sequence + t0 + tid) * geo.value_heads + hv;
    gate = load_gate(in.g, gi, in.gate_fp32);
    beta = __bfloat162float(in.beta[gi]);
  }
  const float prefix = chunk_prefix64(gate, tid, carry);
  if (tid < kChunk) {
    sp[tid] = prefix;
    sbeta[tid] = beta;
    sexp[tid] = expf(prefix);
    scoef[tid] = beta * expf(prefix);
  }
  for (int e = tid; e < kChunk * kDim; e += kPrepareThreads) {
    const int i = e / kDim, d = e % kDim;
    float kv = 0.f, qv = 0.f;
    if (i < valid) {
      const long long off = (((long long)b * geo.sequence + t0 + i) * geo.key_heads + hk) * kDim + d;
      kv = __bfloat162float(in.k[off]);
      qv = __bfloat162float(in.q[off]);
    }
    sK[i * kPad + d] = kv;
    sX[i * kPad + d] = qv;
  }
  __syncthreads();

  // decay-masked K.K^T (strictly lower) and Q.K^T (lower incl. diagonal)
  for (int e = tid; e < kChunk * kChunk; e += kPrepareThreads) {
    const int i = e / kChunk, j = e % kChunk;
    float kk = 0.f, qk = 0.f;
    if (j <= i) {
      for (int d = 0; d < kDim; ++d) {
        const float kj = sK[j * kPad + d];
        kk = fmaf(sK[i * kPad + d], kj, kk);
        qk = fmaf(sX[i * kPad + d], kj, qk);
      }
    }
    const float decay = (j <= i) ? expf(sp[i] - sp[j]) : 0.f;
    sT[i * (kChunk + 1) + j] = (j < i) ? sbeta[i] * kk * decay : 0.f;
    ws.p[block * kChunk * kChunk + e] = __float2bfloat16_rn(qk * decay * kScale);
  }
  __syncthreads();

  // T = (I + A)^-1 by forward substitution, one column per thread, in place
  // (column c of the result only needs rows >= c; entries above the diagonal stay 0).
  // Lock-step rows: at step i every thread c <= i computes T[i][c] from A[i][*] (row i is still
  // original A, since row i entries are only written at step i) and T[j][c] (j < i, final).
  for (int i = 0; i < kChunk; ++i) {
    float value = 0.f;
    if (tid < kChunk) {
      const int c = tid;
      if (c == i) value = 1.f;
      else if (c < i) {
        float acc = 0.f;
        for (int j = c; j < i; ++j) acc = fmaf(sT[i * (kChunk + 1) + j], sT[j * (kChunk + 1) + c], acc);
        value = -acc;
      }
    }
    __syncthreads();     // every read of row i (original A) is done
    if (tid < kChunk) sT[i * (kChunk + 1) + tid] = value;
    __syncthreads();
  }

  // W = T diag(beta exp(p)) K  -> BF16 hi/lo pair
  {
    const int d = tid % kDim, half = tid / kDim;
    for (int r = 0; r < kChunk / 2; ++r) {
      const int i = half * (kChunk / 2) + r;
      float acc = 0.f;
      for (int c = 0; c <= i; ++c) acc = fmaf(sT[i * (kChunk + 1) + c] * scoef[c], sK[c * kPad + d], acc);
      __nv_bfloat16 hi, lo;
      split_bf16(acc, hi, lo);
      ws.w_hi[transposed_index(block, i, d)] = hi;
      ws.w_lo[transposed_index(block, i, d)] = lo;
    }
  }
  __syncthreads();
  // U = T diag(beta) V
  for (int e = tid; e < kChunk * kDim; e += kPrepareThreads) {
    const int i = e / kDim, d = e % kDim;
    float vv = 0.f;
    if (i < valid)
      vv = __bfloat162float(in.v[(((long long)b * geo.sequence + t0 + i) * geo.value_heads + hv) * kDim + d]);
    sX[i * kPad + d] = vv;
  }
  __syncthreads();
  {
    const int d = tid % kDim, half = tid / kDim;
    for (int r = 0; r < kChunk / 2; ++r) {
      const int i = half * (kChunk / 2) + r;
      float acc = 0.f;
      for (int c = 0; c <= i; ++c) acc = fmaf(sT[i * (kChunk + 1) + c] * sbeta[c], sX[c * kPad + d], acc);
      ws.u[block * kChunk * kDim + i * kDim + d] = acc;
    }
  }
  if (tid < kChunk) ws.gates[block * kGateWords + tid] = (tid < valid) ? expf(sp[valid - 1] - sp[tid]) : 0.f;
  if (tid == kChunk) ws.gates[block * kGateWords + kChunk] = expf(sp[valid - 1]);
  if (tid < kChunk) ws.gates[block * kGateWords + kGateQueryScale + tid] = sexp[tid] * kScale;   // query scale
}

// ---------------------------------------------------------------------------------------------
constexpr int kVt = 32;                 // value columns per CTA
constexpr int kWalkThreads = 256;
constexpr int kWalkSmem =
    (kDim * kVt + 3 * kChunk * kPad + kChunk * (kChunk + 1) + 3 * kChunk * kVt + 128) * 4;

__global__ void __launch_bounds__(kWalkThreads)
walk_simt_kernel(Inputs in, Geometry geo, Workspace ws) {
  extern __shared__ float smem[];
  float* sS = smem;                          // [128][32] state tile (key dim, value col)
  float* sW = sS + kDim * kVt;               // [64][129]
  float* sK = sW + kChunk * kPad;            // [64][129]
  float* sQ = sK + kChunk * kPad;            // [64][129]
  float* sP = sQ + kChunk * kPad;            // [64][65]
  float* sU = sP + kChunk * (kChunk + 1);    // [64][32]
  float* sN = sU + kChunk * kVt;             // [64][32]
  float* sNr = sN + kChunk * kVt;            // [64][32]  N * rel
  float* sG = sNr + kChunk * kVt;            // [128]

  const int tid = threadIdx.x;
  const int v0 = (blockIdx.x % (kDim / kVt)) * kVt;
  const int bh = blockIdx.x / (kDim / kVt);
  const int b = bh / geo.value_heads, hv = bh % geo.value_heads;
  const int hk = hv / geo.group();
  const int lane_v = tid % kVt, row0 = tid / kVt;      // row0 in [0,8)

  for (int e = tid; e < kDim * kVt; e += kWalkThreads) {
    const int d = e / kVt, v = e % kVt;
    sS[e] = in.initial ? in.initial[((long long)bh * kDim + d) * kDim + v0 + v] : 0.f;
  }
  const int chunks = geo.chunks();
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int t0 = chunk * kChunk;
    const int valid = min(kChunk, geo.sequence - t0);
    const long long block = (long long)bh * chunks + chunk;
    __syncthreads();
    for (int e = tid; e < kChunk * kDim; e += kWalkThreads) {
      const int i = e / kDim, d = e % kDim;
      const long long off = block * kChunk * kDim + e;
      sW[i * kPad + d] = __bfloat162float(ws.w_hi[transposed_index(block, i, d)]) +
                         __bfloat162float(ws.w_lo[transposed_index(block, i, d)]);
      float kv = 0.f, qv = 0.f;
      if (i < valid) {
        const long long at = (((long long)b * geo.sequence + t0 + i) * geo.key_heads + hk) * kDim + d;
        kv = __bfloat162float(in.k[at]);
        // the scaled query as the tensor-core walk forms it: one BF16 rounding of q * exp(p) / sqrt(128)
        qv = __bfloat162float(__float2bfloat16_rn(__bfloat162float(in.q[at]) * ws.gates[block * kGateWords + kGateQueryScale + i]));
      }
      sQ[i * kPad + d] = qv;
      sK[i * kPad + d] = kv;
    }
    for (int e = tid; e < kChunk * kChunk; e += kWalkThreads)
      sP[(e / kChunk) * (kChunk + 1) + e % kChunk] = __bfloat162float(ws.p[block * kChunk * kChunk + e]);
    for (int e = tid; e < kChunk * kVt; e += kWalkThreads)
      sU[e] = ws.u[block * kChunk * kDim + (e / kVt) * kDim + v0 + e % kVt];
    if (tid < 128) sG[tid] = ws.gates[block * kGateWords + tid];
    __syncthreads();

    // N = U - W S
    for (int r = 0; r < kChunk / 8; ++r) {
      const int i = row0 + 8 * r;
      float acc = 0.f;
      for (int d = 0; d < kDim; ++d) acc = fmaf(sW[i * kPad + d], sS[d * kVt + lane_v], acc);
      const float n = sU[i * kVt + lane_v] - acc;
      sN[i * kVt + lane_v] = n;
      sNr[i * kVt + lane_v] = n * sG[i];
    }
    __syncthreads();
    // O = Qs S + P N   (old state)
    for (int r = 0; r < kChunk / 8; ++r) {
      const int i = row0 + 8 * r;
      float acc = 0.f;
      for (int d = 0; d < kDim; ++d) acc = fmaf(sQ[i * kPad + d], sS[d * kVt + lane_v], acc);
      for (int j = 0; j <= i; ++j) acc = fmaf(sP[i * (kChunk + 1) + j], sN[j * kVt + lane_v], acc);
      if (i < valid)
        in.output[(((long long)b * geo.sequence + t0 + i) * geo.value_heads + hv) * kDim + v0 + lane_v] =
            __float2bfloat16_rn(acc);
    }
    __syncthreads();
    // S <- gamma S + K^T (N * rel)
    const float gamma = sG[kChunk];
    for (int r = 0; r < kDim / 8; ++r) {
      const int d = row0 + 8 * r;
      float acc = gamma * sS[d * kVt + lane_v];
      for (int i = 0; i < kChunk; ++i) acc = fmaf(sK[i * kPad + d], sNr[i * kVt + lane_v], acc);
      sS[d * kVt + lane_v] = acc;
    }
  }
  __syncthreads();
  if (in.final_state)
    for (int e = tid; e < kDim * kVt; e += kWalkThreads)
      in.final_state[((long long)bh * kDim + e / kVt) * kDim + v0 + e % kVt] = sS[e];
}

}  // namespace

int configure_simt() {
  cudaError_t e = cudaFuncSetAttribute(prepare_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kPrepareSmem);
  if (e != cudaSuccess) return int(e);
  e = cudaFuncSetAttribute(walk_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWalkSmem);
  return int(e);
}

int launch_prepare_simt(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  dim3 grid((unsigned)geo.blocks());
  prepare_simt_kernel<<<grid, kPrepareThreads, kPrepareSmem, stream>>>(in, geo, ws);
  return int(cudaGetLastError());
}

int launch_walk_simt(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  dim3 grid((unsigned)(geo.batch * geo.value_heads * (kDim / kVt)));
  walk_simt_kernel<<<grid, kWalkThreads, kWalkSmem, stream>>>(in, geo, ws);
  return int(cudaGetLastError());
}

}  // namespace gdn_sm100
