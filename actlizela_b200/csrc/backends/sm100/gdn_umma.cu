// Tensor-core implementation (configuration "umma") of the two stages of the chunked
// gated-delta-rule forward for sm_100a: tcgen05.mma with accumulators and A operands in tensor
// memory, B operands in 128-byte-swizzled shared memory staged by TMA, mbarrier hand-offs.
//
// Orientation.  Every product is arranged so that its M dimension is 128 (one TMEM lane per row):
// the state is held TRANSPOSED, St[v][k] (value index on lanes, key index on columns), so that
//   (W S)^T = St W^T     (Q S)^T = St Q^T     (P N)^T = N^T P^T     St += (N*rel)^T K
// all have M = 128 value rows, and St / N^T are consumed as A operands straight from tensor memory.
//
// Precision.  All tcgen05 MMAs are kind::f16 with BF16 operands and FP32 accumulation (the small block products
// of the triangular inverse run as 3xTF32 mma.sync tiles, see the prepare kernel).  Quantities on the
// path to the final state are carried as BF16 pairs x ~= hi + lo (16 significant bits):
// the triangular inverse T (scaled by beta, exp(prefix)), W, the state operand of W S and N*rel.
// K, V, Q are exact BF16 inputs.  U is never rounded (FP32 from accumulator to register).
// Output-side operands (P, scaled Q, N for P N, the state operand of Q S) are single BF16.
//
// Math reference: the WY chunk form of the reference project (tests/wy_cpu.py:44-88;
// prepare/state/output kernels csrc/gdn_chunk/gdn_wy_ppu.cu:7-292), re-derived in transposed form.
#include "gdn_common.cuh"
#include "umma.cuh"

namespace gdn_sm100 {
using namespace ptx;

// =============================================================================== host: tensor maps
int TensorMapEncoder::init() {
  if (encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult query;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query);
  if (e != cudaSuccess) return int(e);
  if (query != cudaDriverEntryPointSuccess || !fn) return int(cudaErrorNotSupported);
  encode = reinterpret_cast<Fn>(fn);
  return 0;
}

int TensorMapEncoder::bf16_2d(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                              uint32_t box_rows) const {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                      elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(cudaErrorInvalidValue);
}

int TensorMapEncoder::bf16_4d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t d3, uint32_t box_rows_d2) const {
  const cuuint64_t dims[4] = {d0, d1, d2, d3};
  const cuuint64_t strides[3] = {d0 * 2, d0 * d1 * 2, d0 * d1 * d2 * 2};
  const cuuint32_t box[4] = {64, 1, box_rows_d2, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                      elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(cudaErrorInvalidValue);
}

int TensorMapEncoder::f32_2d(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                             uint32_t box_rows) const {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {32, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box,
                      elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(cudaErrorInvalidValue);
}

TensorMapEncoder& tensor_map_encoder() {
  static TensorMapEncoder encoder;
  return encoder;
}

namespace {

// Heads (batch x value head, summed over launches) that a parallel walk really split [0] / walked with one CTA
// because a sub-segment does not decay or a token is not a contraction [1]; read by read_walk_plan_counts.
__device__ int g_walk_plan_counts[2];

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kBox = 8192;            // one TMA box: 64 rows x 128 bytes
constexpr uint32_t kIdescN64 = idesc_bf16(128, 64, false, false);      // A K-major (smem or TMEM), B K-major
constexpr uint32_t kIdescN64AT = idesc_bf16(128, 64, true, false);     // A MN-major (transposed smem tile)
constexpr uint32_t kIdescN128BT = idesc_bf16(128, 128, false, true);   // B MN-major

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed FP32 pairs (two IEEE round-to-nearest operations per instruction on sm_100): the arithmetic of the walk's
// chain warps is bound by instruction issue, and these halve its floating-point instruction count bit for bit.
#define GDN_F32X2(name, op)                                                                                      \
  __device__ __forceinline__ void name(float& x0, float& x1, float a0, float a1, float b0, float b1) {          \
    asm("{\n\t.reg .b64 a, b, c;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\t" op                       \
        ".rn.f32x2 c, a, b;\n\tmov.b64 {%0, %1}, c;\n\t}"                                                       \
        : "=f"(x0), "=f"(x1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));                                              \
  }
GDN_F32X2(add2, "add")
GDN_F32X2(sub2, "sub")
GDN_F32X2(mul2, "mul")
#undef GDN_F32X2
// d += a b for one m16n8k8 tile with FP32-grade accuracy from TF32 tensor-core products: a ~ ah + al, b ~ bh + bl
// (both parts TF32), d += ah bh + ah bl + al bh (the 3xTF32 scheme the reference uses for these merges,
// tests/wy_cpu.py:10-18).  Fragment layout of mma.m16n8k8: g = lane / 4, t = lane % 4;
// a = {A[g][t], A[g+8][t], A[g][t+4], A[g+8][t+4]}, b = {B[t][g], B[t+4][g]}, d = {D[g][2t], D[g][2t+1], D[g+8][2t], D[g+8][2t+1]}.
__device__ __forceinline__ void mma_tf32x3(float (&d)[4], const float (&a)[4], const float (&b)[2]) {
  // The high part is the operand with its 13 low mantissa bits cleared (a TF32 value), the low part the exact FP32
  // remainder, of which the tensor core reads the leading TF32 bits: about 2^-20 relative in all, below the
  // 16 significant bits the inverse is later stored with.  Logic and add instructions: the conversion unit, the
  // kernel's busiest pipe, stays free for the BF16 packing.
  uint32_t ah[4], al[4], bh[2], bl[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ah[i] = __float_as_uint(a[i]) & 0xffffe000u;
    al[i] = __float_as_uint(a[i] - __uint_as_float(ah[i]));
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    bh[i] = __float_as_uint(b[i]) & 0xffffe000u;
    bl[i] = __float_as_uint(b[i] - __uint_as_float(bh[i]));
  }
#define GDN_MMA_TF32(A, B)                                                                              \
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, " \
               "{%8, %9}, {%0, %1, %2, %3};"                                                             \
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])                                          \
               : "r"(A[0]), "r"(A[1]), "r"(A[2]), "r"(A[3]), "r"(B[0]), "r"(B[1]))
  GDN_MMA_TF32(al, bh);
  GDN_MMA_TF32(ah, bl);
  GDN_MMA_TF32(ah, bh);
#undef GDN_MMA_TF32
}
// One m16n8 tile of D = A B over k in [0, kdim): A row-major with pitch lda (rows a_row0 + {g, g+8}), B row-major with
// pitch ldb (column b_col0 + g); both in shared memory.
__device__ __forceinline__ void tile_product_tf32x3(float (&d)[4], const float* a, int lda, const float* b, int ldb,
                                                    int kdim, int g, int t) {
#pragma unroll
  for (int k0 = 0; k0 < kdim; k0 += 8) {
    const float av[4] = {a[g * lda + k0 + t], a[(g + 8) * lda + k0 + t], a[g * lda + k0 + t + 4], a[(g + 8) * lda + k0 + t + 4]};
    const float bv[2] = {b[(k0 + t) * ldb + g], b[(k0 + t + 4) * ldb + g]};
    mma_tf32x3(d, av, bv);
  }
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// ================================================================================= prepare kernel
// One CTA per (batch, value head, chunk) block, 256 threads, THREE CTAs per SM (at most 80 registers, 67 KB of
// shared memory, 128 tensor-memory columns): the phases of a block are serial and latency bound, so the
// throughput comes from the blocks in flight.  A warp owns the TMEM lane quarter (warp & 3) and, of every
// accumulator it reads, the column half (warp >> 2).
//   phase 1  TMA: Q, K chunk tiles (key head of the group) and V tile; gate prefix by two warps
//   phase 2  D1[128x64] = [Q;K] K^T                                  (one tcgen05 product, 8 instructions)
//   phase 3  rows 0..63  -> P = tril(QK^T * decay)/sqrt(128) -> BF16 -> workspace
//            rows 64..127-> A = tril(beta_i KK^T * decay, -1) -> shared (FP32);
//            the diagonal k_i.k_i decides whether token i is a contraction (word 65 of the gate vector)
//   phase 4  T = (I+A)^-1 IN PLACE, blocked: four 16x16 diagonal solves in FP32 registers, then
//            T21 = -T22 (A21 T11) at block size 16 and 32 as 3xTF32 mma.sync tiles (the blocked scheme and the
//            TF32x3 merges of the reference's tests/wy_cpu.py:10-41)
//            T diag(beta exp(p)) and T diag(beta) -> BF16 hi/lo K-major tiles: the first pair over the dead Q
//            boxes, the second over T itself (every thread holds its part of T in registers by then)
//   phase 5  W^T = K^T (T diag(beta exp p))^T (into the columns D1 occupied),  U^T = V^T (T diag(beta))^T
//            (A = transposed K / V tiles)
//   phase 6  accumulators -> registers -> workspace.  W is stored transposed, [key dim][token]: a thread owns one
//            row and stages its 32 tokens as 16-byte pieces in swizzled tiles that leave through TMA stores; U is
//            token-major and leaves straight from registers (a warp writes 128 contiguous bytes per token)
struct PrepLayout {
  static constexpr int kQ0 = 0, kK0 = kBox, kQ1 = 2 * kBox, kK1 = 3 * kBox;   // [Q;K] stacked, two K atoms
  static constexpr int kV0 = 4 * kBox, kV1 = 5 * kBox;
  static constexpr int kLd = 68;                           // row pitch (floats) of the FP32 64x64 matrix
  static constexpr int kAT = 6 * kBox;                     // float [64][68]: A, then T in place
  static constexpr int kTwH = kQ0, kTwL = kQ1;             // written after phase 4, when Q and the scratch are dead
  static constexpr int kTuH = kAT, kTuL = kAT + kBox;      // written once T sits in registers
  static constexpr int kX = kQ0;                           // block products of the inverse, on the dead Q box
  static constexpr int kStageWH = 0, kStageWL = 2 * kBox;  // phase 6: W^T hi / lo tiles [128][64] over the Q/K boxes
  static constexpr int kLdX = 20, kLdX3 = 36;
  static constexpr int kVec = kAT + 64 * kLd * 4;          // float [4][64]: pl2, beta, beta*exp(p), exp(p)/sqrt(128)
  static constexpr int kBars = kVec + 4 * 64 * 4;          // 2 mbarriers, tmem slot, abort flag, carry
  static constexpr int kTotal = kBars + 64;
  static_assert(2 * kBox <= 64 * kLd * 4 && kAT % 1024 == 0, "the U pair of T tiles must fit on T, box aligned");
  static_assert(32 * kLdX3 * 4 <= kBox && 32 * kLdX * 4 <= kBox, "block-product scratch must fit in one Q box");
};
constexpr int kPrepThreads = 256;
constexpr int kPrepSmem = PrepLayout::kTotal + 1024;
constexpr int kPrepTmemCols = 128;   // D1 [0,64), later W^T;  U^T [64,128)
static_assert(3 * (kPrepSmem + 1024) <= 227 * 1024, "three prepare CTAs must fit in one SM's shared memory");

#ifdef GDN_SM100_PHASE_TIMING
#define GDN_PSTAMP(slot) \
  if (tid == 0) ws.gates[block * kGateWords + 80 + (slot)] = float((clock64() - t_begin) & 0xffffff)
#else
#define GDN_PSTAMP(slot)
#endif

// Fused variant (kFused): the tiles come from the packed projection rows (tm_q is a 2-D map over them, tm_k the 4-D
// map of the normalised-key plane that the walk reads); Q and K rows are L2-normalised in shared memory with the
// arithmetic of the separate input-preparation kernel (16 lanes per row), gate and beta are activated on load.
template <bool kFused>
__global__ void __launch_bounds__(kPrepThreads, 3)
prepare_umma_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_wh,
                    const __grid_constant__ CUtensorMap tm_wl, Inputs in, Geometry geo, Workspace ws) {
  // Indexing the declared array (no integer round trip) keeps these accesses in the shared state space.
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* sm = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  using L = PrepLayout;
  float* sAT = reinterpret_cast<float*>(sm + L::kAT);
  float* sX = reinterpret_cast<float*>(sm + L::kX);
  float* s_pl2 = reinterpret_cast<float*>(sm + L::kVec);
  float* s_beta = s_pl2 + 64;
  float* s_coefw = s_beta + 64;
  float* s_qscale = s_coefw + 64;
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(sm + L::kBars);
  uint64_t* bar_mma = bar_tma + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* carry = reinterpret_cast<float*>(tmem_slot + 2);
  const AbortFlag abort{abort_word};

  const int tid = threadIdx.x, warp = tid >> 5;
  const int chunks = geo.chunks(), seg_chunks = geo.segment_chunks();
  int chunk = geo.chunk_begin + blockIdx.x % seg_chunks;      // chunk index inside its sequence
  int bh = blockIdx.x / seg_chunks;
  if (!geo.varlen) {
    // Block order = reverse of the order in which the walk consumes the blocks: the walk's CTAs (one per
    // (batch, head) and parallel sub-segment) all start at the first chunk of their sub-segment, so the blocks
    // prepared LAST are the leading chunks of every sub-segment of every head, and the walk finds them in L2.
    // The grid covers heads x sub-segments x longest sub-segment; a slot behind a shorter sub-segment's end is empty.
    const int parallel = geo.parallel > 1 ? geo.parallel : 1;
    // (The cut is an even one; the walk's own cut, sub_segment_begin, differs from it by a few chunks at most.)
    const int longest = (seg_chunks + parallel - 1) / parallel;
    const int units = geo.batch * geo.value_heads * parallel;
    const int offset = longest - 1 - int(blockIdx.x) / units, unit = int(blockIdx.x) % units;
    const int sub = unit % parallel;
    const int sub_begin = int((long long)seg_chunks * sub / parallel), sub_end = int((long long)seg_chunks * (sub + 1) / parallel);
    if (sub_begin + offset >= sub_end) return;
    bh = unit / parallel;
    chunk = geo.chunk_begin + sub_begin + offset;
  }
  const int b = bh / geo.value_heads, hv = bh % geo.value_heads;     // packed mode: bh = hv, b = 0
  const int hk = hv / geo.group();
  int t0 = chunk * kChunk, t_end = geo.sequence;
  long long block = (long long)bh * chunks + chunk;
  if (geo.varlen) {
    // packed sequences: the grid runs over (value head, global chunk); rows behind the sequence end belong to the
    // next sequence and are neutralised by beta = 0 / zero gate weights exactly like zero-filled padding rows
    const int gchunk = chunk;
    const int* prefix = geo.varlen + geo.batch + 1;
    if (gchunk >= prefix[geo.batch]) return;     // grid sized by an upper bound of the chunk count (device offsets)
    const int seq = varlen_sequence_of(prefix, geo.batch, gchunk);
    chunk = gchunk - prefix[seq];
    t0 = geo.varlen[seq] + chunk * kChunk;
    t_end = geo.varlen[seq + 1];
    block = (long long)hv * chunks + gchunk;
  }
  const int valid = min(kChunk, t_end - t0);
#ifdef GDN_SM100_PHASE_TIMING
  const long long t_begin = clock64();
#endif

  if (tid == 0) {
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    *abort_word = 0;
    fence_barrier_init();
    // the input tiles do not depend on tensor memory: start them before the allocation
    mbar_arrive_expect_tx(bar_tma, 6 * kBox);
    if (kFused) {
      // packed rows [q heads | k heads | v heads]; rows behind the batch element's end belong to the next one
      // (or read as zero behind the last) and are neutralised by beta = 0 / zero gate weights
      const int row = b * geo.sequence + t0;
      const int xq = hk * kDim, xk = (geo.key_heads + hk) * kDim, xv = (2 * geo.key_heads + hv) * kDim;
      tma_load_2d(sm + L::kQ0, &tm_q, bar_tma, xq, row);
      tma_load_2d(sm + L::kQ1, &tm_q, bar_tma, xq + 64, row);
      tma_load_2d(sm + L::kK0, &tm_q, bar_tma, xk, row);
      tma_load_2d(sm + L::kK1, &tm_q, bar_tma, xk + 64, row);
      tma_load_2d(sm + L::kV0, &tm_q, bar_tma, xv, row);
      tma_load_2d(sm + L::kV1, &tm_q, bar_tma, xv + 64, row);
    } else {
      tma_load_4d(sm + L::kQ0, &tm_q, bar_tma, 0, hk, t0, b);
      tma_load_4d(sm + L::kQ1, &tm_q, bar_tma, 64, hk, t0, b);
      tma_load_4d(sm + L::kK0, &tm_k, bar_tma, 0, hk, t0, b);
      tma_load_4d(sm + L::kK1, &tm_k, bar_tma, 64, hk, t0, b);
      tma_load_4d(sm + L::kV0, &tm_v, bar_tma, 0, hv, t0, b);
      tma_load_4d(sm + L::kV1, &tm_v, bar_tma, 64, hv, t0, b);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kPrepTmemCols);
    tmem_relinquish();
  }
  float gate = 0.f, beta = 0.f;
  if (tid < valid) {
    const long long gi = ((long long)b * geo.sequence + t0 + tid) * geo.value_heads + hv;
    if (kFused) {
      // g = -exp(A_log) softplus(a + dt_bias) (z > 20 branch), beta = sigmoid(b) rounded to BF16
      const float z = __bfloat162float(in.act_a[gi]) + in.dt_bias[hv];
      gate = -expf(in.a_log[hv]) * (z > 20.f ? z : log1pf(expf(z)));
      beta = __bfloat162float(__float2bfloat16_rn(1.f / (1.f + expf(-__bfloat162float(in.act_b[gi])))));
    } else {
      gate = load_gate(in.g, gi, in.gate_fp32);
      beta = __bfloat162float(in.beta[gi]);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  GDN_PSTAMP(0);

  const float prefix = chunk_prefix64(gate, tid, carry);   // contains a __syncthreads
  if (tid < kChunk) {
    const float e = exp2f(prefix * kLog2e);
    s_pl2[tid] = prefix * kLog2e;
    s_beta[tid] = beta;
    s_coefw[tid] = beta * e;
    s_qscale[tid] = e * kScale;
  }
  __syncthreads();

  // ---- phase 2: D1 = [Q;K] K^T
  bool ok = mbar_wait(bar_tma, 0, abort, 1, chunk);
  GDN_PSTAMP(1);
  if (kFused) {
    // L2-normalise the 64 Q and 64 K rows in place: 16 lanes per row (8 BF16 = one swizzled 16-byte slot each),
    // 16 rows per pass; x * rsqrt(sum x^2 + 1e-6) rounded to BF16
    if (ok) {
      const int lane16 = tid & 15;
#pragma unroll
      for (int pass = 0; pass < 8; ++pass) {
        const int r = pass * 16 + (tid >> 4), row = r & 63;
        uint8_t* slot = sm + (r < 64 ? (lane16 < 8 ? L::kQ0 : L::kQ1) : (lane16 < 8 ? L::kK0 : L::kK1)) + row * 128 +
                        (((lane16 & 7) ^ (row & 7)) << 4);
        const uint4 x = *reinterpret_cast<const uint4*>(slot);
        const float f[8] = {bf16_lo(x.x), bf16_hi(x.x), bf16_lo(x.y), bf16_hi(x.y),
                            bf16_lo(x.z), bf16_hi(x.z), bf16_lo(x.w), bf16_hi(x.w)};
        float square = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) square = fmaf(f[e], f[e], square);
#pragma unroll
        for (int d = 8; d; d >>= 1) square += __shfl_xor_sync(0xffffffffu, square, d, 16);
        const float factor = rsqrtf(square + 1e-6f);
        *reinterpret_cast<uint4*>(slot) = make_uint4(pack_bf16(f[0] * factor, f[1] * factor), pack_bf16(f[2] * factor, f[3] * factor),
                                                     pack_bf16(f[4] * factor, f[5] * factor), pack_bf16(f[6] * factor, f[7] * factor));
      }
      fence_proxy_async_smem();
    }
    __syncthreads();
    // the walk reads the normalised queries and keys: one CTA per key-head group stores the tiles (rows behind T
    // are clipped); tm_v doubles as the map of the normalised-query plane in this variant
    if (tid == 0 && ok && hv % geo.group() == 0) {
      tma_store_4d(&tm_k, sm + L::kK0, 0, hk, t0, b);
      tma_store_4d(&tm_k, sm + L::kK1, 64, hk, t0, b);
      tma_store_4d(&tm_v, sm + L::kQ0, 0, hk, t0, b);
      tma_store_4d(&tm_v, sm + L::kQ1, 64, hk, t0, b);
      tma_store_commit();
    }
  }
  if (tid == 0 && ok) {
    tc_fence_after();
    const uint32_t base = smem_u32(sm);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t a = base + (ks < 4 ? L::kQ0 : L::kQ1) + (ks & 3) * 32;
      const uint32_t bb = base + (ks < 4 ? L::kK0 : L::kK1) + (ks & 3) * 32;
      mma_ss(tmem + 0, smem_desc(a, 16, 1024), smem_desc(bb, 16, 1024), kIdescN64, ks > 0);
    }
    mma_commit(bar_mma);
  }
  ok = ok && mbar_wait(bar_mma, 0, abort, 2, chunk);
  tc_fence_after();
  GDN_PSTAMP(2);

  // ---- phase 3: masks and decays on D1
  // warp -> TMEM lane quarter (warp & 3) and column half (warp >> 2) of the 64 columns
  const int quarter = warp & 3, chalf = warp >> 2;
  const int lrow = quarter * 32 + (tid & 31);          // accumulator row owned by this thread
  const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16);
  bool not_contraction = false;
  if (ok) {
    const int i = lrow & 63;
    const float pi = s_pl2[i], bi = s_beta[i];
    uint32_t d[2][16];
    tmem_ld16(taddr + chalf * 32, d[0]);
    tmem_ld16(taddr + chalf * 32 + 16, d[1]);
    tmem_wait_ld();
    float kk = 0.f;                                      // k_i . k_i when the diagonal lies in this column half
#pragma unroll
    for (int piece = 0; piece < 2; ++piece) {
      const int j0 = chalf * 32 + piece * 16;
      if (j0 > (i | 31)) {
        // the whole piece lies above the diagonal for every row of this warp (rows (i & ~31) .. (i | 31)): zeros
        if (lrow < 64) {
          uint4* dst = reinterpret_cast<uint4*>(ws.p + (block * kChunk + i) * kChunk + j0);
          dst[0] = dst[1] = make_uint4(0u, 0u, 0u, 0u);
        } else {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<float4*>(sAT + i * L::kLd + j0 + q4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        continue;
      }
      float pj[16];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float4 t = *reinterpret_cast<const float4*>(s_pl2 + j0 + q4 * 4);
        pj[q4 * 4] = t.x; pj[q4 * 4 + 1] = t.y; pj[q4 * 4 + 2] = t.z; pj[q4 * 4 + 3] = t.w;
      }
      if (lrow < 64) {
        uint32_t packed[8];
#pragma unroll
        for (int jj = 0; jj < 16; jj += 2) {
          const int j = j0 + jj;
          const float a0 = (j <= i) ? __uint_as_float(d[piece][jj]) * fast_exp2(pi - pj[jj]) * kScale : 0.f;
          const float a1 = (j + 1 <= i) ? __uint_as_float(d[piece][jj + 1]) * fast_exp2(pi - pj[jj + 1]) * kScale : 0.f;
          packed[jj >> 1] = pack_bf16(a0, a1);
        }
        uint4* dst = reinterpret_cast<uint4*>(ws.p + (block * kChunk + i) * kChunk + j0);
        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      } else {
        float* arow = sAT + i * L::kLd + j0;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float a[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int jj = q4 * 4 + e;
            a[e] = (j0 + jj < i) ? bi * __uint_as_float(d[piece][jj]) * fast_exp2(pi - pj[jj]) : 0.f;
            if (j0 + jj == i) kk = __uint_as_float(d[piece][jj]);
          }
          *reinterpret_cast<float4*>(arow + q4 * 4) = make_float4(a[0], a[1], a[2], a[3]);
        }
      }
    }
    tc_fence_before();      // D1's columns are overwritten by the W^T product once every thread has passed the barriers
    // token i multiplies the state by exp(g_i) (I - beta_i k_i k_i^T): a contraction iff 0 <= beta_i |k_i|^2 <= 2
    if (lrow >= 64) not_contraction = !(bi >= 0.f && bi * kk <= 2.f);
  }
  if (kFused && tid == 0) tma_store_wait_read();     // the Q and K tiles' stores have left shared memory: the
                                                     // inverse's scratch and the T tiles reuse the Q boxes from here on
  const int chunk_not_contraction = __syncthreads_or(not_contraction);
  ok = __syncthreads_and(ok);                  // uniform from here on: the warp-level barrier below needs that
  GDN_PSTAMP(3);

  // ---- phase 4: T = (I+A)^-1 in place, blocked 16 -> 32 -> 64, all in FP32 on the CUDA cores
  // level 1: the four 16x16 diagonal blocks, one column per thread (left-looking, in registers); the 16 threads
  // of a block sit in one warp and overwrite the block only after all of them have read it
  if (ok && tid < 64) {
    const int blk = tid >> 4, c = tid & 15;
    float* a0 = sAT + (blk * 16) * L::kLd + blk * 16;
    float x[16];
    float4 cur[4], nxt[4] = {};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      // fetch the next row's lower-triangle part before the dependent FMA chain of this row
#pragma unroll
      for (int j4 = 0; j4 < i + 1 && i + 1 < 16; j4 += 4)
        nxt[j4 >> 2] = *reinterpret_cast<const float4*>(a0 + (i + 1) * L::kLd + j4);
      float acc0 = (i == c) ? 1.f : 0.f, acc1 = 0.f;
#pragma unroll
      for (int j4 = 0; j4 < i; j4 += 4) {
        const float4 a = cur[j4 >> 2];
        if (j4 + 0 < i) acc0 = fmaf(-a.x, x[j4 + 0], acc0);
        if (j4 + 1 < i) acc1 = fmaf(-a.y, x[j4 + 1], acc1);
        if (j4 + 2 < i) acc0 = fmaf(-a.z, x[j4 + 2], acc0);
        if (j4 + 3 < i) acc1 = fmaf(-a.w, x[j4 + 3], acc1);
      }
      x[i] = acc0 + acc1;
#pragma unroll
      for (int q = 0; q < 4; ++q) cur[q] = nxt[q];
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 16; ++i) a0[i * L::kLd + c] = x[i];
  }
  __syncthreads();
  GDN_PSTAMP(7);
  // level 2: inside each 32x32 diagonal block, T21 = -T22 (A21 T11) with 16x16 blocks, written where A21 was.
  // Levels 2 and 3 are small dense products: they run on the tensor cores as m16n8k8 TF32 tiles with the 3xTF32
  // split (FP32-grade accuracy), one tile per warp, operands read from shared memory one word per lane; as FP32 FMAs
  // with vector loads they made up more than half of the kernel's shared-memory traffic, which is what bounds it.
  {
    const int lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int big = warp >> 1, nt = warp & 1, o = big * 32;        // warps 0..3: (diagonal block, 8-column tile)
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok && warp < 4) {
      tile_product_tf32x3(c, sAT + (o + 16) * L::kLd + o, L::kLd, sAT + o * L::kLd + o + nt * 8, L::kLd, 16, g, t);
      *reinterpret_cast<float2*>(sX + (big * 16 + g) * L::kLdX + nt * 8 + 2 * t) = make_float2(c[0], c[1]);
      *reinterpret_cast<float2*>(sX + (big * 16 + g + 8) * L::kLdX + nt * 8 + 2 * t) = make_float2(c[2], c[3]);
    }
    __syncthreads();
    if (ok && warp < 4) {
      c[0] = c[1] = c[2] = c[3] = 0.f;
      tile_product_tf32x3(c, sAT + (o + 16) * L::kLd + o + 16, L::kLd, sX + big * 16 * L::kLdX + nt * 8, L::kLdX, 16, g, t);
      *reinterpret_cast<float2*>(sAT + (o + 16 + g) * L::kLd + o + nt * 8 + 2 * t) = make_float2(-c[0], -c[1]);
      *reinterpret_cast<float2*>(sAT + (o + 16 + g + 8) * L::kLd + o + nt * 8 + 2 * t) = make_float2(-c[2], -c[3]);
    }
  }
  __syncthreads();
  GDN_PSTAMP(8);
  // level 3: T21 = -T22 (A21 T11) with 32x32 blocks: eight tiles, one per warp
  {
    const int lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mt = warp >> 2, nt = warp & 3;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok) {
      tile_product_tf32x3(c, sAT + (32 + mt * 16) * L::kLd, L::kLd, sAT + nt * 8, L::kLd, 32, g, t);
      *reinterpret_cast<float2*>(sX + (mt * 16 + g) * L::kLdX3 + nt * 8 + 2 * t) = make_float2(c[0], c[1]);
      *reinterpret_cast<float2*>(sX + (mt * 16 + g + 8) * L::kLdX3 + nt * 8 + 2 * t) = make_float2(c[2], c[3]);
    }
    __syncthreads();
    if (ok) {
      c[0] = c[1] = c[2] = c[3] = 0.f;
      tile_product_tf32x3(c, sAT + (32 + mt * 16) * L::kLd + 32, L::kLd, sX + nt * 8, L::kLdX3, 32, g, t);
      *reinterpret_cast<float2*>(sAT + (32 + mt * 16 + g) * L::kLd + nt * 8 + 2 * t) = make_float2(-c[0], -c[1]);
      *reinterpret_cast<float2*>(sAT + (32 + mt * 16 + g + 8) * L::kLd + nt * 8 + 2 * t) = make_float2(-c[2], -c[3]);
    }
  }
  __syncthreads();
  GDN_PSTAMP(9);
  // T diag(beta exp p) and T diag(beta) as BF16 hi/lo K-major tiles; thread -> row i, sixteen columns (conflict-free:
  // the row pitch of 68 words spreads eight consecutive rows over all banks, the tile rows are swizzled).
  // The W pair goes to the Q boxes at once; the U pair overwrites T, so it waits until every thread has read its part.
  {
    const int i = tid & 63, c0 = (tid >> 6) * 16;      // a warp's lanes: consecutive rows, the same columns
    uint32_t uh[8], ul[8];
    if (ok) {
#pragma unroll
      for (int g8 = 0; g8 < 2; ++g8) {
        const int c = c0 + g8 * 8;
        float t[8], cw[8], cu[8];
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4) {
          const float4 tv = *reinterpret_cast<const float4*>(sAT + i * L::kLd + c + q4 * 4);
          const float4 wv = *reinterpret_cast<const float4*>(s_coefw + c + q4 * 4);
          const float4 uv = *reinterpret_cast<const float4*>(s_beta + c + q4 * 4);
          t[q4 * 4] = tv.x; t[q4 * 4 + 1] = tv.y; t[q4 * 4 + 2] = tv.z; t[q4 * 4 + 3] = tv.w;
          cw[q4 * 4] = wv.x; cw[q4 * 4 + 1] = wv.y; cw[q4 * 4 + 2] = wv.z; cw[q4 * 4 + 3] = wv.w;
          cu[q4 * 4] = uv.x; cu[q4 * 4 + 1] = uv.y; cu[q4 * 4 + 2] = uv.z; cu[q4 * 4 + 3] = uv.w;
        }
        uint32_t wh[4], wl[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float w0 = t[e] * cw[e], w1 = t[e + 1] * cw[e + 1];
          const float u0 = t[e] * cu[e], u1 = t[e + 1] * cu[e + 1];
          const uint32_t hw = pack_bf16(w0, w1), hu = pack_bf16(u0, u1);
          wh[e >> 1] = hw;
          wl[e >> 1] = pack_bf16(w0 - bf16_lo(hw), w1 - bf16_hi(hw));
          uh[g8 * 4 + (e >> 1)] = hu;
          ul[g8 * 4 + (e >> 1)] = pack_bf16(u0 - bf16_lo(hu), u1 - bf16_hi(hu));
        }
        const int off = i * 128 + (((c >> 3) ^ (i & 7)) << 4);
        *reinterpret_cast<uint4*>(sm + L::kTwH + off) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
        *reinterpret_cast<uint4*>(sm + L::kTwL + off) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
      }
    }
    __syncthreads();
    if (ok) {
#pragma unroll
      for (int g8 = 0; g8 < 2; ++g8) {
        const int c = c0 + g8 * 8;
        const int off = i * 128 + (((c >> 3) ^ (i & 7)) << 4);
        *reinterpret_cast<uint4*>(sm + L::kTuH + off) = make_uint4(uh[g8 * 4], uh[g8 * 4 + 1], uh[g8 * 4 + 2], uh[g8 * 4 + 3]);
        *reinterpret_cast<uint4*>(sm + L::kTuL + off) = make_uint4(ul[g8 * 4], ul[g8 * 4 + 1], ul[g8 * 4 + 2], ul[g8 * 4 + 3]);
      }
      fence_proxy_async_smem();
    }
  }
  __syncthreads();
  GDN_PSTAMP(4);

  // ---- phase 5: W^T (into D1's columns, which every thread has read) and U^T
  if (tid == 0 && ok) {
    tc_fence_after();
    const uint32_t base = smem_u32(sm);
#pragma unroll
    for (int part = 0; part < 2; ++part) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t a = smem_desc(base + L::kK0 + ks * 2048, L::kK1 - L::kK0, 1024);
        const uint64_t bb = smem_desc(base + (part ? L::kTwL : L::kTwH) + ks * 32, 16, 1024);
        mma_ss(tmem + 0, a, bb, kIdescN64AT, (part | ks) != 0);
      }
    }
#pragma unroll
    for (int part = 0; part < 2; ++part) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t a = smem_desc(base + L::kV0 + ks * 2048, L::kV1 - L::kV0, 1024);
        const uint64_t bb = smem_desc(base + (part ? L::kTuL : L::kTuH) + ks * 32, 16, 1024);
        mma_ss(tmem + 64, a, bb, kIdescN64AT, (part | ks) != 0);
      }
    }
    mma_commit(bar_mma);
  }
  // the gate vector does not depend on the products: write it while they run
  if (ok) {
    const float last = s_pl2[valid - 1];
    if (tid < kChunk) ws.gates[block * kGateWords + tid] = (tid < valid) ? fast_exp2(last - s_pl2[tid]) : 0.f;
    if (tid == kChunk) ws.gates[block * kGateWords + kChunk] = fast_exp2(last);
    if (tid == kChunk + 1) ws.gates[block * kGateWords + kChunk + 1] = chunk_not_contraction ? 1.f : 0.f;
    if (tid >= 128 && tid < 128 + kChunk) ws.gates[block * kGateWords + kGateQueryScale + tid - 128] = s_qscale[tid - 128];
  }
  ok = ok && mbar_wait(bar_mma, 1, abort, 3, chunk);
  tc_fence_after();
  GDN_PSTAMP(5);

  // ---- phase 6: W (hi/lo) and U leave for the workspace; lrow is the key (W) / value (U) index.
  // W^T: the thread's 32 tokens are contiguous in its row; they are staged as 16-byte pieces in two
  // 128-byte-swizzled tiles [128 keys][64 tokens] on the dead input boxes and leave through two TMA stores
  // (16-byte stores from registers to global would touch 32 lines per warp instruction).
  // U: token-major [64][128] FP32, what the walk's chain warps read one value per lane: a warp's 32 lanes write
  // 128 contiguous bytes per token straight from registers.
  if (ok) {
    uint8_t* stage_hi = sm + L::kStageWH + lrow * 128;
    uint8_t* stage_lo = sm + L::kStageWL + lrow * 128;
    float* dst_u = ws.u + block * (kChunk * kDim) + lrow;
#pragma unroll
    for (int piece = 0; piece < 2; ++piece) {
      const int tk0 = chalf * 32 + piece * 16;
      uint32_t dw[16], du[16];
      tmem_ld16(taddr + tk0, dw);
      tmem_ld16(taddr + 64 + tk0, du);
      tmem_wait_ld();
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int jj = 0; jj < 16; jj += 2) {
        const float w0 = __uint_as_float(dw[jj]), w1 = __uint_as_float(dw[jj + 1]);
        const uint32_t h = pack_bf16(w0, w1);
        hi[jj >> 1] = h;
        lo[jj >> 1] = pack_bf16(w0 - bf16_lo(h), w1 - bf16_hi(h));
      }
#pragma unroll
      for (int h8 = 0; h8 < 2; ++h8) {          // eight tokens = one 16-byte slot of the swizzled row
        const int slot = (((tk0 >> 3) + h8) ^ (lrow & 7)) << 4;
        *reinterpret_cast<uint4*>(stage_hi + slot) = make_uint4(hi[h8 * 4], hi[h8 * 4 + 1], hi[h8 * 4 + 2], hi[h8 * 4 + 3]);
        *reinterpret_cast<uint4*>(stage_lo + slot) = make_uint4(lo[h8 * 4], lo[h8 * 4 + 1], lo[h8 * 4 + 2], lo[h8 * 4 + 3]);
      }
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) dst_u[(tk0 + jj) * kDim] = __uint_as_float(du[jj]);
    }
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (tid == 0 && ok) {
    const int row = int(block * kDim);
    tma_store_2d(&tm_wh, sm + L::kStageWH, 0, row);
    tma_store_2d(&tm_wl, sm + L::kStageWL, 0, row);
    tma_store_commit();
    tma_store_wait_read();
  }
  GDN_PSTAMP(6);
  if (!ok) {
    for (int i = 0; i < 20; ++i) __nanosleep(100000);   // let copies in flight land before the CTA leaves
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kPrepTmemCols);
}
#undef GDN_PSTAMP

// ==================================================================================== walk kernel
// One CTA per (batch, value head), or per (batch, value head, parallel sub-segment): see the comment above the
// kernel; 512 threads, one CTA per SM.  Tensor memory (512 columns):
//   ACC_S [  0,128)  St FP32 accumulator (pre-scaled by the chunk decay before the update MMA)
//   OP_SH [128,192)  St BF16 hi, packed pairs      OP_SL [192,256)  St BF16 lo
//   ACC_X [256,384)  S_hi^T [W_hi ; W_lo]^T, with S_lo^T W_hi^T added to the first half:
//           [256,320) (W_hi S)^T   [320,384) (W_lo S_hi)^T
//         after N = U - W S has been formed, the columns are reused for the N operands of the
//         16-token group ks:  (N*rel) hi at 256+16ks, lo at 256+16ks+8,  N (BF16) at 320+16ks
//   ACC_O [384,448) and [448,512)  O^T = S_hi^T Qs^T + N^T P^T, alternating by chunk: the epilogue drains one
//         while the next chunk's products fill the other
// Per chunk: 16 instructions for W S (N = 128 and 64), on which the chain waits; 8 for S Qs and 4 for P N, issued
// behind the commits the chain waits for; 8 for the state update (N = 128).
// Roles: warp 0 MMA issuer and warp 1 TMA producer (the lowest warp ids: their short instruction streams
//        sit on the critical path and must not queue behind the arithmetic of the chain warps);
//        warps 4-11 state chain: a warp owns the 32 TMEM lanes of quarter (warp & 3) and, of every tile it
//        touches, one column half.  Both chain steps are signalled in two halves so that the MMA issuer
//        starts on the first half of the K range while the second half is still being written.
//        warps 2-3 query scaling: the Q tile of a ring stage becomes Qs = Q exp(p) / sqrt(128) in place (one BF16
//        rounding, a row's scale from the gate vector) before the issuer reads it for the state part of the output;
//        warps 12-15 output epilogue.
struct WalkLayout {
  // one ring stage: W^T hi and lo tiles [128 key lines][64 tokens] (MN-major B operand of the wide product, the
  // lo tile one 16 KB tile behind the hi tile), Q as two K-major boxes (scaled in place to Qs by the scaling
  // warps), K as two boxes, P, the gate vector (768 bytes)
  static constexpr int kWH = 0, kWL = 2 * kBox;
  static constexpr int kQS0 = 4 * kBox, kQS1 = 5 * kBox;
  static constexpr int kK = 6 * kBox, kP = 8 * kBox;
  static constexpr int kGates = 9 * kBox;
  static constexpr int kStage = 9 * kBox + 1024;
  static constexpr int kStages = 2;
  static constexpr int kTxBytes = 9 * kBox + kGateWords * 4;
  static constexpr int kOut = kStages * kStage;           // two staging tiles [64 tokens][128 values] BF16
  static constexpr int kBars = kOut + 4 * kBox;
  static constexpr int kTotal = kBars + 256;
};
constexpr int kMmaWarp = 0, kTmaWarp = 1, kScaleWarp0 = 2, kScaleWarps = 2, kChainWarp0 = 4, kChainWarps = 8, kOutWarp0 = 12;
constexpr int kWalkThreads = 512;
constexpr int kWalkSmem = WalkLayout::kTotal + 1024;
constexpr uint32_t kAccS = 0, kOpSH = 128, kOpSL = 192, kAccX = 256, kAccO = 384;   // ACC_O: two buffers of 64
constexpr uint32_t kIdescN64BT = idesc_bf16(128, 64, false, true);     // B MN-major, N = 64

#ifdef GDN_SM100_PHASE_TIMING
#define GDN_STAMP(slot)                                                                        \
  if (tid == kChainWarp0 * 32) ws.gates[(block0 + c) * kGateWords + 96 + (slot)] = float((clock64() - t_begin) & 0xffffff)
#define GDN_MSTAMP(slot) ws.gates[(block0 + c) * kGateWords + 104 + (slot)] = float((clock64() - t_begin) & 0xffffff)
#define GDN_OSTAMP(slot)                                                                       \
  if (tid == kOutWarp0 * 32) ws.gates[(block0 + c) * kGateWords + 112 + (slot)] = float((clock64() - t_begin) & 0xffffff)
#else
#define GDN_STAMP(slot)
#define GDN_MSTAMP(slot)
#define GDN_OSTAMP(slot)
#endif

// First chunk boundary of a sub-segment at which the decay accumulated since the sub-segment's start is below
// exp(-40): returns the number of leading chunks an incoming state still reaches (1..count), or -1 when the decay
// never gets that far inside the sub-segment.  `not_contraction` collects word 65 of every chunk's gate vector.
// Warp-collective; every caller with the same (first block, count) gets the same answer: two CTAs rely on that.
__device__ __forceinline__ int decay_reach(const float* gates, long long first_block, int count, int lane,
                                           bool& not_contraction) {
  float total = 0.f;
  int reach = -1;
  bool flagged = false;
  for (int c0 = 0; c0 < count; c0 += 128) {
    // four independent loads in flight per lane, then four scan steps of 32 chunks
    float2 w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * 32 + lane;
      w[u] = c < count ? *reinterpret_cast<const float2*>(gates + (first_block + c) * kGateWords + kChunk)
                       : make_float2(1.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * 32 + lane;
      float x = c < count ? log2f(w[u].x) : 0.f;
      flagged |= w[u].y != 0.f;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      const unsigned below = __ballot_sync(0xffffffffu, c < count && total + x < kDecayedLog2);
      if (below && reach < 0) reach = c0 + u * 32 + __ffs(below);
      total += __shfl_sync(0xffffffffu, x, 31);
    }
  }
  not_contraction |= __any_sync(0xffffffffu, flagged);
  return reach;
}

// Shortest suffix of a chunk range whose accumulated decay is below exp(-40) and whose tokens are all contractions:
// returns its length in chunks (1..count), or -1 when there is none.  A walk of that suffix from a zero state ends
// in the state the whole range ends in from ANY incoming state, to exp(-40) of that state.  Warp-collective.
__device__ __forceinline__ int decay_suffix(const float* gates, long long first_block, int count, int lane) {
  float total = 0.f;
  bool flagged = false;
  for (int done = 0; done < count; done += 32) {
    const int back = done + lane;                         // chunks behind the range's last one
    const float2 w = back < count
        ? *reinterpret_cast<const float2*>(gates + (first_block + count - 1 - back) * kGateWords + kChunk)
        : make_float2(1.f, 0.f);
    float x = back < count ? log2f(w.x) : 0.f;
    flagged |= w.y != 0.f;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    const unsigned below = __ballot_sync(0xffffffffu, back < count && total + x < kDecayedLog2);
    if (below) {
      // flags of chunks in front of the suffix (higher lanes) do not matter
      const int length = __ffs(below);
      const unsigned bad = __ballot_sync(0xffffffffu, flagged) & (0xffffffffu >> (32 - length));
      return bad ? -1 : done + length;
    }
    if (__any_sync(0xffffffffu, flagged)) return -1;      // (so `flagged` only ever holds this step's chunks)
    total += __shfl_sync(0xffffffffu, x, 31);
  }
  return -1;
}

// Parallel sub-segments (Geometry::parallel = P > 1): the launch's chunk range of every (batch, value head) is cut
// into P sub-segments and the grid holds P CTAs per head.  CTA r walks sub-segment r from a ZERO state (r = 0 from
// the true incoming state) and then carries on into the leading chunks of sub-segment r + 1, those that its state
// still reaches with a weight above exp(-40), writing their output rows; CTA r + 1 computes the same number from the
// same gate words and does not store those rows.  This is exact to exp(-40) of the state when every sub-segment
// behind the first decays below exp(-40) within its own length and every token transition exp(g)(I - beta k k^T) is
// a contraction (0 <= beta |k|^2 <= 2; the prepare kernel records violations).  A head for which that does not hold
// is walked by its first CTA alone over the whole range, as without the split; its other CTAs leave at once.
// The last sub-segment's CTA (or the single CTA) writes the outgoing state.
__global__ void __launch_bounds__(kWalkThreads, 1)
walk_umma_kernel(const __grid_constant__ CUtensorMap tm_wh, const __grid_constant__ CUtensorMap tm_wl,
                 const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_out,
                 Inputs in, Geometry geo, Workspace ws) {
  // Indexing the declared array (no integer round trip) keeps these accesses in the shared state space.
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* sm = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  using L = WalkLayout;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L::kBars);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + L::kStages;         // [kStages]
  uint64_t* bar_ops = bars + 2 * L::kStages;   // [2] state operands written, first / second K half
  uint64_t* bar_opn = bar_ops + 2;             // [2] N operands written, first / second token half
  uint64_t* bar_ws = bar_ops + 4;              // wide product complete
  uint64_t* bar_s = bar_ops + 5;               // state update complete
  uint64_t* bar_o = bar_ops + 6;               // output accumulator complete
  uint64_t* bar_ofree = bar_ops + 10;          // [2] output accumulator (c & 1) drained (one arrival per output warp)
  uint64_t* bar_staged = bar_ops + 8;          // output tile staged in shared memory (one arrival per output warp)
  uint64_t* bar_stfree = bar_ops + 9;          // an older output store has finished reading its staging tile
  uint64_t* bar_qs = bar_ops + 12;             // [2] the ring stage's Q tile has been scaled (one arrival per scaling warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ops + 14);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* limit_slot = reinterpret_cast<int*>(tmem_slot + 2);      // [4]: [0] chunks of a cut-short walk, [1] transition is zero, [2] suffix of the offset pass
  const AbortFlag abort{abort_word};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int parallel = geo.parallel > 1 ? geo.parallel : 1;
  // Pair pass (kWalkPair): the grid holds two CTAs per (batch, value head); the first set runs the offset pass
  // (kWalkTail), the second the transition pass (kWalkHomogeneous) from an identity state made here.
  const bool pair_pass = (in.walk_flags & kWalkPair) != 0;
  const int heads = geo.batch * geo.value_heads;
  const int unit = blockIdx.x / parallel, sub = blockIdx.x % parallel;
  const int bh = pair_pass ? unit % heads : unit;
  const int flags = pair_pass ? (unit >= heads ? kWalkHomogeneous : kWalkTail) : in.walk_flags;
  int b = bh / geo.value_heads;
  const int hv = bh % geo.value_heads;
  const int hk = hv / geo.group();
  int chunks = geo.segment_chunks();                 // this launch walks `chunks` chunks from token t_first on
  int t_first = geo.chunk_begin * kChunk, tail_valid = kChunk;
  long long block0 = (long long)bh * geo.chunks() + geo.chunk_begin;
  if (geo.varlen) {
    // packed sequences: one CTA per (sequence, value head); states are indexed by bh = sequence * Hv + hv
    const int seq = b;
    const int* prefix = geo.varlen + geo.batch + 1;
    chunks = prefix[seq + 1] - prefix[seq];
    t_first = geo.varlen[seq];
    tail_valid = geo.varlen[seq + 1] - t_first - (chunks - 1) * kChunk;     // rows of the sequence's last chunk
    block0 = (long long)hv * geo.total_chunks + prefix[seq];
    b = 0;
  }
  const float* state_in = geo.first_segment() ? in.initial : ws.carry;
  float* state_out = geo.last_segment() ? in.final_state : ws.carry;
  if (sub > 0) state_in = nullptr;
  bool identity_in = false;
  if (pair_pass) {
    // final_state is the pair block [2][B][Hv][128][128]: transition matrices first, offsets behind them
    state_in = nullptr;
    identity_in = (flags & kWalkHomogeneous) != 0;
    state_out = in.final_state + ((flags & kWalkTail) ? (long long)heads * kDim * kDim : 0);
  }
#ifdef GDN_SM100_PHASE_TIMING
  const long long t_begin = clock64();
#endif

  if (tid == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(bar_ops, kChainWarps);
    mbar_init(bar_ops + 1, kChainWarps);
    mbar_init(bar_opn, kChainWarps);
    mbar_init(bar_opn + 1, kChainWarps);
    mbar_init(bar_ws, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_init(bar_ofree, 4);
    mbar_init(bar_ofree + 1, 4);
    mbar_init(bar_staged, 4);
    mbar_init(bar_stfree, 1);
    mbar_init(bar_qs, kScaleWarps);
    mbar_init(bar_qs + 1, kScaleWarps);
    *abort_word = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if ((flags & kWalkUntilDecayed) && warp == kTmaWarp) {
    // first chunk boundary at which the accumulated decay is below exp(-40): 32 chunks per step, the per-chunk
    // decay exp(p_last) is word 64 of the chunk's gate vector
    float total = 0.f;
    int stop = chunks;
    for (int c0 = 0; c0 < chunks && stop == chunks; c0 += 32) {
      const int c = c0 + lane;
      float x = c < chunks ? log2f(ws.gates[(block0 + c) * kGateWords + kChunk]) : 0.f;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      const unsigned below = __ballot_sync(0xffffffffu, c < chunks && total + x < kDecayedLog2);
      if (below) stop = c0 + __ffs(below);          // chunks [0, stop) are walked
      total += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) *limit_slot = stop;
  }
  if ((flags & kWalkHomogeneous) && warp == kTmaWarp) {
    // transition pass: a range that decays below exp(-40) (all tokens contractions) has a transition matrix
    // below exp(-40) in norm; it is returned as exact zeros without walking
    bool flagged = false;
    const int reach = decay_reach(ws.gates, block0, chunks, lane, flagged);
    if (lane == 0) limit_slot[1] = (reach >= 0 && !flagged) ? 1 : 0;
  }
  if ((flags & kWalkTail) && warp == kTmaWarp) {
    const int keep = decay_suffix(ws.gates, block0, chunks, lane);
    if (lane == 0) limit_slot[2] = keep > 0 ? keep : chunks;        // no such suffix: the whole range from zero
  }
  int* reach_slot = limit_slot + 4;             // [8] per sub-segment: chunks an incoming state reaches, -1 = invalid
  if (parallel > 1 && warp >= 1 && warp < parallel) {
    // plan (see the comment above the kernel): warp r scans sub-segment r (sub_segment_begin gives the cut)
    const int n = chunks;
    const int r0 = sub_segment_begin(n, warp, parallel), r1 = sub_segment_begin(n, warp + 1, parallel);
    bool flagged = false;
    const int reach = decay_reach(ws.gates, block0 + r0, r1 - r0, lane, flagged);
    if (lane == 0) reach_slot[warp] = flagged ? -1 : reach;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (flags & kWalkUntilDecayed) chunks = *limit_slot;
  if ((flags & kWalkHomogeneous) && limit_slot[1]) {
    chunks = 0;
    state_in = nullptr;           // zeros go into tensor memory and straight out as the transition matrix
    identity_in = false;
  }
  int unstored = 0;                          // leading chunks whose output rows the previous sub-segment's CTA writes
  if (flags & kWalkTail) {
    // offset pass: only the suffix that determines the outgoing state, from zero, no output rows
    const int keep = limit_slot[2];
    t_first += (chunks - keep) * kChunk;
    block0 += chunks - keep;
    chunks = unstored = keep;
    state_in = nullptr;
  }
  if (parallel > 1) {
    const int n = chunks;
    bool serial = false;
    for (int r = 1; r < parallel; ++r) serial |= reach_slot[r] < 0;
    if (tid == 0 && sub == 0) atomicAdd(&g_walk_plan_counts[serial ? 1 : 0], 1);
    if (serial) {
      chunks = sub == 0 ? n : 0;             // the head's first CTA walks the whole range alone
      if (sub != 0) state_out = nullptr;
    } else {
      const int c0 = sub_segment_begin(n, sub, parallel), c1 = sub_segment_begin(n, sub + 1, parallel);
      chunks = c1 - c0 + (sub + 1 < parallel ? reach_slot[sub + 1] : 0);
      t_first += c0 * kChunk;
      block0 += c0;
      unstored = sub == 0 ? 0 : reach_slot[sub];
      if (sub != parallel - 1) state_out = nullptr;
    }
  }

  if (warp >= kChainWarp0 && warp < kChainWarp0 + kChainWarps) {
    // ------------------------------------------------------------------ state chain
    const int quarter = warp & 3, half = (warp - kChainWarp0) >> 2;
    const int v = quarter * 32 + lane;                     // value row = TMEM lane
    const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16);
    {
      const float* init = state_in ? state_in + (long long)bh * kDim * kDim + v : nullptr;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t vals[32];
        const int k0 = half * 64 + part * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          vals[j] = init ? __float_as_uint(init[(k0 + j) * kDim]) : ((identity_in && k0 + j == v) ? __float_as_uint(1.f) : 0u);
        tmem_st32(taddr + kAccS + k0, vals);
      }
      tmem_wait_st();
    }
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int s = c % L::kStages;
      const float* gates = reinterpret_cast<const float*>(sm + s * L::kStage + L::kGates);
      // U plane, token-major: the 32 lanes of the warp read 128 contiguous bytes per token
      const float* urow = ws.u + ((block0 + c) * kChunk + half * 32) * kDim + v;
      if (c + 1 < chunks)      // pull the next chunk's U rows of this warp towards L2
        asm volatile("prefetch.global.L2 [%0];" ::"l"(urow + kChunk * kDim + lane * kDim - lane));

      if (c > 0) ok = mbar_wait(bar_s, (c - 1) & 1, abort, 10, c);
      ok = ok && mbar_wait(full + s, (c / L::kStages) & 1, abort, 11, c);
      if (!ok) break;
      tc_fence_after();
      GDN_STAMP(0);
      const float gamma = gates[kChunk];
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t d[32], hi[16], lo[16];
        const int k0 = half * 64 + part * 32;
        tmem_ld32(taddr + kAccS + k0, d);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float s0 = __uint_as_float(d[j]), s1 = __uint_as_float(d[j + 1]);
          const uint32_t h = pack_bf16(s0, s1);
          hi[j >> 1] = h;
          float l0, l1, g0, g1;
          sub2(l0, l1, s0, s1, bf16_lo(h), bf16_hi(h));
          lo[j >> 1] = pack_bf16(l0, l1);
          mul2(g0, g1, s0, s1, gamma, gamma);
          d[j] = __float_as_uint(g0);
          d[j + 1] = __float_as_uint(g1);
        }
        tmem_st16(taddr + kOpSH + (k0 >> 1), hi);
        tmem_st16(taddr + kOpSL + (k0 >> 1), lo);
        tmem_st32(taddr + kAccS + k0, d);
        tmem_wait_st();
        tc_fence_before();
        // the products overwrite one O^T buffer (last used two chunks ago) and read the ring stage: this warp
        // vouches for both before its first arrival, so the issuer has a single wait in front of them
        if (part == 0 && c > 1) ok = mbar_wait(bar_ofree + (c & 1), ((c >> 1) - 1) & 1, abort, 14, c);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ops + part);
      }
      if (!ok) break;
      GDN_STAMP(1);

      float u[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) u[i] = (flags & kWalkHomogeneous) ? 0.f : __ldg(urow + i * kDim);

      ok = mbar_wait(bar_ws, c & 1, abort, 12, c);
      if (!ok) break;
      tc_fence_after();
      GDN_STAMP(2);
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int ks = half * 2 + part;                     // 16-token group
        uint32_t dh[16], dl[16], nh[8], nl[8], n16[8];
        tmem_ld16(taddr + kAccX + ks * 16, dh);
        tmem_ld16(taddr + kAccX + 64 + ks * 16, dl);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const int i = ks * 16 + j;
          float z0, z1, n0, n1, r0, r1, e0, e1;
          add2(z0, z1, __uint_as_float(dh[j]), __uint_as_float(dh[j + 1]), __uint_as_float(dl[j]), __uint_as_float(dl[j + 1]));
          sub2(n0, n1, u[part * 16 + j], u[part * 16 + j + 1], z0, z1);
          mul2(r0, r1, n0, n1, gates[i], gates[i + 1]);
          const uint32_t h = pack_bf16(r0, r1);
          nh[j >> 1] = h;
          sub2(e0, e1, r0, r1, bf16_lo(h), bf16_hi(h));
          nl[j >> 1] = pack_bf16(e0, e1);
          n16[j >> 1] = pack_bf16(n0, n1);
        }
        tmem_st8(taddr + kAccX + ks * 16, nh);
        tmem_st8(taddr + kAccX + ks * 16 + 8, nl);
        tmem_st8(taddr + kAccX + 64 + ks * 16, n16);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_opn + part);
      }
      GDN_STAMP(3);
    }
    if (ok && chunks > 0) ok = mbar_wait(bar_s, (chunks - 1) & 1, abort, 13, chunks);
    if (ok && state_out) {
      tc_fence_after();
      float* fin = state_out + (long long)bh * kDim * kDim + v;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t d[32];
        const int k0 = half * 64 + part * 32;
        tmem_ld32(taddr + kAccS + k0, d);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) fin[(k0 + j) * kDim] = __uint_as_float(d[j]);
      }
    }
  }  else if (warp >= kOutWarp0) {
    // ------------------------------------------------------------------ output epilogue
    const int quarter = warp - kOutWarp0;
    const int v = quarter * 32 + lane;
    const uint32_t tbase = tmem + (uint32_t(quarter * 32) << 16) + kAccO;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      ok = mbar_wait(bar_o, c & 1, abort, 20, c);
      if (!ok) break;
      tc_fence_after();
      GDN_OSTAMP(0);
      const uint32_t taddr = tbase + (c & 1) * 64;
      uint32_t o[64];
      {
        uint32_t d0[32], d1[32];
        tmem_ld32(taddr, d0);
        tmem_ld32(taddr + 32, d1);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          o[j] = d0[j];
          o[32 + j] = d1[j];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ofree + (c & 1));
      GDN_OSTAMP(1);
      if (c < unstored) continue;
      const int cs = c - unstored;           // count of stored tiles: staging buffers and their barriers follow it
      if (geo.varlen && c == chunks - 1 && tail_valid < kChunk) {
        // packed mode, ragged end of a sequence: the rows behind it belong to the next sequence, so the tile
        // cannot leave through a clipping TMA store; this is the sequence's last chunk, nothing follows it
        __nv_bfloat16* out = in.output + ((long long)(t_first + c * kChunk) * geo.value_heads + hv) * kDim + v;
        const long long row = (long long)geo.value_heads * kDim;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < tail_valid) out[i * row] = __float2bfloat16_rn(__uint_as_float(o[i]));
        break;
      }
      // stage the tile as two 128-byte-swizzled boxes [token][64 values] and hand it to a TMA store,
      // which also clips the rows of a tail chunk at the sequence end
      uint8_t* stage = sm + L::kOut + (cs & 1) * 2 * kBox + (v >> 6) * kBox + ((v & 7) << 1);
      const int chunk16 = (v & 63) >> 3;
      // the store that used this buffer two chunks ago has been read out (signalled one chunk ago)
      if (cs > 0) ok = mbar_wait(bar_stfree, (cs - 1) & 1, abort, 21, c);
      if (!ok) break;
#pragma unroll
      for (int i = 0; i < 64; ++i)
        *reinterpret_cast<__nv_bfloat16*>(stage + i * 128 + ((chunk16 ^ (i & 7)) << 4)) =
            __float2bfloat16_rn(__uint_as_float(o[i]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_staged);
      if (tid == kOutWarp0 * 32) {
        ok = mbar_wait(bar_staged, cs & 1, abort, 22, c);
        if (!ok) break;
        const uint8_t* tile = sm + L::kOut + (cs & 1) * 2 * kBox;
        tma_store_4d(&tm_out, tile, 0, hv, t_first + c * kChunk, b);
        tma_store_4d(&tm_out, tile + kBox, 64, hv, t_first + c * kChunk, b);
        tma_store_commit();
        tma_store_wait_read_keep1();
        mbar_arrive(bar_stfree);
      }
      GDN_OSTAMP(2);
    }
    if (tid == kOutWarp0 * 32) tma_store_wait_all();
  } else if (warp >= kScaleWarp0 && warp < kScaleWarp0 + kScaleWarps) {
    // ------------------------------------------------------------------ query scaling
    // 64 threads turn the 64 x 128 Q tile of a ring stage into Qs in place: 16 pieces of 16 bytes per thread; a
    // row's 16 pieces lie in two swizzled boxes (columns 0..63 and 64..127)
    const int t64 = tid - kScaleWarp0 * 32;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int s = c % L::kStages;
      ok = mbar_wait(full + s, (c / L::kStages) & 1, abort, 50, c);
      if (!ok) break;
      uint8_t* st = sm + s * L::kStage;
      const float* scale = reinterpret_cast<const float*>(st + L::kGates) + kGateQueryScale;
#pragma unroll 4
      for (int it = 0; it < 16; ++it) {
        const int piece = it * 64 + t64, row = piece >> 4, col16 = piece & 15;
        uint4* at = reinterpret_cast<uint4*>(st + (col16 < 8 ? L::kQS0 : L::kQS1) + row * 128 + (((col16 & 7) ^ (row & 7)) << 4));
        const float f = scale[row];
        const uint4 v = *at;
        uint4 o;
        o.x = pack_bf16(bf16_lo(v.x) * f, bf16_hi(v.x) * f);
        o.y = pack_bf16(bf16_lo(v.y) * f, bf16_hi(v.y) * f);
        o.z = pack_bf16(bf16_lo(v.z) * f, bf16_hi(v.z) * f);
        o.w = pack_bf16(bf16_lo(v.w) * f, bf16_hi(v.w) * f);
        *at = o;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_qs + s);
    }
  } else if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_wh);
      prefetch_tensormap(&tm_wl);
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_p);
      for (int c = 0; c < chunks; ++c) {
        if ((flags & kWalkSelftestStall) && c > 0) break;       // failure-detection self-test only
        const int s = c % L::kStages;
        if (c >= L::kStages && !mbar_wait(empty + s, ((c / L::kStages) - 1) & 1, abort, 30, c)) break;
        uint8_t* st = sm + s * L::kStage;
        const int row = int((block0 + c) * kChunk);
        mbar_arrive_expect_tx(full + s, L::kTxBytes);
        bulk_load(st + L::kGates, ws.gates + (block0 + c) * kGateWords, kGateWords * 4, full + s);
        tma_load_2d(st + L::kWH, &tm_wh, full + s, 0, 2 * row);       // transposed planes: 128 rows per block
        tma_load_2d(st + L::kWL, &tm_wl, full + s, 0, 2 * row);
        tma_load_4d(st + L::kQS0, &tm_q, full + s, 0, hk, t_first + c * kChunk, b);
        tma_load_4d(st + L::kQS1, &tm_q, full + s, 64, hk, t_first + c * kChunk, b);
        tma_load_4d(st + L::kK, &tm_k, full + s, 0, hk, t_first + c * kChunk, b);
        tma_load_4d(st + L::kK + kBox, &tm_k, full + s, 64, hk, t_first + c * kChunk, b);
        tma_load_2d(st + L::kP, &tm_p, full + s, 0, row);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // The issuing thread is a latency-bound scalar program: the loop holds no data-dependent branch but one check
    // of the wait results per chunk (a wait that gave up lets the rest of that chunk's instructions run on stale
    // operands, which is harmless: the launch is already failed), and the base addresses are broadcast so that
    // the compiler knows they are warp-uniform.
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t st0 = __shfl_sync(0xffffffffu, smem_u32(sm), 0);
    if (lane == 0) {
      bool ok = true;
      // Descriptors of ring stage 0; stage 1 is a constant further on (the start-address field counts 16-byte units).
      static_assert(L::kStages == 2 && L::kStage % 16 == 0, "descriptor arithmetic below assumes a two-stage ring");
      const uint64_t dW = smem_desc(st0 + L::kWH, L::kWL - L::kWH, 1024);      // MN-major: 64-token groups hi | lo
      const uint64_t dQ0 = smem_desc(st0 + L::kQS0, 16, 1024), dQ1 = smem_desc(st0 + L::kQS1, 16, 1024);
      const uint64_t dK = smem_desc(st0 + L::kK, kBox, 1024), dP = smem_desc(st0 + L::kP, 16, 1024);
      for (int c = 0; c < chunks && ok; ++c) {
        const uint64_t stage = uint64_t((c & 1) * (L::kStage >> 4));
        const uint64_t wd = dW + stage, q0 = dQ0 + stage, q1 = dQ1 + stage, kd = dK + stage, pd = dP + stage;
        const uint32_t acc_o = tm + kAccO + (c & 1) * 64;
        // St [W_hi | W_lo] with St ~ SH + SL (the SL pass only against W_hi, added to the first half).  The B
        // operand is the transposed W tile: key index on the 128-byte lines (K), tokens contiguous (N); one K
        // step of 16 keys is 2048 bytes.  K steps {0,1,4,5} of the split become available first, {2,3,6,7}
        // second.  The chain waits for this product only; the state part of the output, St Qs^T, reads the same
        // operands and is issued behind the commit, so that it runs while the chain warps form N.
        ok = mbar_wait(bar_ops, c & 1, abort, 41, c);
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int ks = (q >> 1) * 4 + (q & 1);
          const uint64_t bdesc = wd + uint64_t(ks * 128);
          mma_ts(tm + kAccX, tm + kOpSH + ks * 8, bdesc, kIdescN128BT, q != 0);
          mma_ts(tm + kAccX, tm + kOpSL + ks * 8, bdesc, kIdescN64BT, 1);
        }
        ok &= mbar_wait(bar_ops + 1, c & 1, abort, 41, c);
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int ks = (q >> 1) * 4 + 2 + (q & 1);
          const uint64_t bdesc = wd + uint64_t(ks * 128);
          mma_ts(tm + kAccX, tm + kOpSH + ks * 8, bdesc, kIdescN128BT, 1);
          mma_ts(tm + kAccX, tm + kOpSL + ks * 8, bdesc, kIdescN64BT, 1);
        }
        mma_commit(bar_ws);
        ok &= mbar_wait(bar_qs + (c & 1), (c >> 1) & 1, abort, 44, c);     // scaled long ago: the tile landed a chunk ahead
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ts(acc_o, tm + kOpSH + ks * 8, ((ks >> 2) ? q1 : q0) + uint64_t((ks & 3) * 2), kIdescN64, ks != 0);
        // St += (N*rel)^T K (accumulator already holds gamma * St); token groups {0,2} first, {1,3} second
        ok &= mbar_wait(bar_opn, c & 1, abort, 43, c);
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int ks = h * 2;
          const uint64_t kdesc = kd + uint64_t(ks * 128);                              // +2048 bytes per K step
          mma_ts(tm + kAccS, tm + kAccX + ks * 16, kdesc, kIdescN128BT, 1);
          mma_ts(tm + kAccS, tm + kAccX + ks * 16 + 8, kdesc, kIdescN128BT, 1);
        }
        ok &= mbar_wait(bar_opn + 1, c & 1, abort, 43, c);
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int ks = h * 2 + 1;
          const uint64_t kdesc = kd + uint64_t(ks * 128);
          mma_ts(tm + kAccS, tm + kAccX + ks * 16, kdesc, kIdescN128BT, 1);
          mma_ts(tm + kAccS, tm + kAccX + ks * 16 + 8, kdesc, kIdescN128BT, 1);
        }
        mma_commit(bar_s);
        // O^T += N^T P^T behind the state update: the next chunk's split waits for that, not for the output
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(acc_o, tm + kAccX + 64 + ks * 16, pd + uint64_t(ks * 2), kIdescN64, 1);
        mma_commit(bar_o);
        mma_commit(empty + (c & 1));
      }
    }
    __syncwarp();
  }
  if (abort.raised()) {
    for (int i = 0; i < 20; ++i) __nanosleep(100000);   // let copies in flight land before the CTA leaves
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
}
#undef GDN_STAMP
#undef GDN_MSTAMP
#undef GDN_OSTAMP

}  // namespace

// ======================================================================================= launchers
int configure_umma() {
  if (int rc = tensor_map_encoder().init()) return rc;
  cudaError_t e = cudaFuncSetAttribute(prepare_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem);
  if (e != cudaSuccess) return int(e);
  e = cudaFuncSetAttribute(prepare_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem);
  if (e != cudaSuccess) return int(e);
  e = cudaFuncSetAttribute(walk_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWalkSmem);
  return int(e);
}

int launch_prepare_umma(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  TensorMapEncoder& enc = tensor_map_encoder();
  if (int rc = enc.init()) return rc;
  CUtensorMap tm_q, tm_k, tm_v;
  const bool fused = in.mixed != nullptr;
  if (fused) {
    if (geo.varlen) return int(cudaErrorInvalidValue);
    // one 2-D map over the packed projection rows; the 4-D map of the normalised-key plane is the store target
    if (int rc = enc.bf16_2d(&tm_q, in.mixed, uint64_t(in.mixed_stride), uint64_t(geo.batch) * geo.sequence, kChunk)) return rc;
    if (int rc = enc.bf16_4d(&tm_k, in.k_norm, kDim, geo.key_heads, geo.sequence, geo.batch, kChunk)) return rc;
    if (int rc = enc.bf16_4d(&tm_v, in.q_norm, kDim, geo.key_heads, geo.sequence, geo.batch, kChunk)) return rc;
  } else {
    if (int rc = enc.bf16_4d(&tm_q, in.q, kDim, geo.key_heads, geo.sequence, geo.varlen ? 1 : geo.batch, kChunk)) return rc;
    if (int rc = enc.bf16_4d(&tm_k, in.k, kDim, geo.key_heads, geo.sequence, geo.varlen ? 1 : geo.batch, kChunk)) return rc;
    if (int rc = enc.bf16_4d(&tm_v, in.v, kDim, geo.value_heads, geo.sequence, geo.varlen ? 1 : geo.batch, kChunk)) return rc;
  }
  // W^T planes: [blocks * 128 key rows][64 tokens], one 128-row box per block (the walk loads the same boxes)
  CUtensorMap tm_wh, tm_wl;
  const uint64_t plane_rows = uint64_t(geo.blocks()) * kDim;
  if (int rc = enc.bf16_2d(&tm_wh, ws.w_hi, kChunk, plane_rows, kDim)) return rc;
  if (int rc = enc.bf16_2d(&tm_wl, ws.w_lo, kChunk, plane_rows, kDim)) return rc;
  const int parallel = geo.parallel > 1 ? geo.parallel : 1;
  const unsigned grid = geo.varlen
      ? (unsigned)((long long)geo.value_heads * geo.segment_chunks())
      : (unsigned)((long long)geo.batch * geo.value_heads * parallel * ((geo.segment_chunks() + parallel - 1) / parallel));
  if (fused)
    prepare_umma_kernel<true><<<grid, kPrepThreads, kPrepSmem, stream>>>(tm_q, tm_k, tm_v, tm_wh, tm_wl, in, geo, ws);
  else
    prepare_umma_kernel<false><<<grid, kPrepThreads, kPrepSmem, stream>>>(tm_q, tm_k, tm_v, tm_wh, tm_wl, in, geo, ws);
  return int(cudaGetLastError());
}
int launch_prepare_fused(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  if (!in.mixed || !in.act_a || !in.act_b || !in.a_log || !in.dt_bias || !in.k_norm || !in.q_norm)
    return int(cudaErrorInvalidValue);
  return launch_prepare_umma(in, geo, ws, stream);
}

int launch_walk_umma(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  TensorMapEncoder& enc = tensor_map_encoder();
  if (int rc = enc.init()) return rc;
  const uint64_t rows = uint64_t(geo.blocks()) * kChunk;
  CUtensorMap tm_wh, tm_wl, tm_q, tm_k, tm_p, tm_out;
  if (int rc = enc.bf16_4d(&tm_out, in.output, kDim, geo.value_heads, geo.sequence, geo.varlen ? 1 : geo.batch, kChunk)) return rc;
  // W^T planes: [blocks * 128 key rows][64 tokens], one 128-row box per block
  if (int rc = enc.bf16_2d(&tm_wh, ws.w_hi, kChunk, 2 * rows, kDim)) return rc;
  if (int rc = enc.bf16_2d(&tm_wl, ws.w_lo, kChunk, 2 * rows, kDim)) return rc;
  if (int rc = enc.bf16_4d(&tm_q, in.q, kDim, geo.key_heads, geo.sequence, geo.varlen ? 1 : geo.batch, kChunk)) return rc;
  if (int rc = enc.bf16_4d(&tm_k, in.k, kDim, geo.key_heads, geo.sequence, geo.varlen ? 1 : geo.batch, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_p, ws.p, kChunk, rows, kChunk)) return rc;
  const int parallel = geo.parallel > 1 ? geo.parallel : 1;
  if (parallel > 1 && (geo.varlen || in.walk_flags || parallel > geo.segment_chunks())) return int(cudaErrorInvalidValue);
  if ((in.walk_flags & kWalkSelftestStall) && (in.walk_flags != kWalkSelftestStall || geo.varlen)) return int(cudaErrorInvalidValue);
  if ((in.walk_flags & (kWalkTail | kWalkPair)) &&
      ((in.walk_flags != kWalkTail && in.walk_flags != kWalkPair) || parallel > 1 || geo.varlen || !geo.first_segment() ||
       !geo.last_segment() || !in.final_state))
    return int(cudaErrorInvalidValue);
  const int per_head = (in.walk_flags & kWalkPair) ? 2 : parallel;
  walk_umma_kernel<<<geo.batch * geo.value_heads * per_head, kWalkThreads, kWalkSmem, stream>>>(
      tm_wh, tm_wl, tm_q, tm_k, tm_p, tm_out, in, geo, ws);
  return int(cudaGetLastError());
}

namespace {
// One warp waits, through the bounded wait every kernel of this file uses, on an mbarrier that nothing ever
// completes.  The wait must give up, record (code 1, block 0, site 99, chunk `tag`) in the status word and let
// the kernel end.
__global__ void wait_timeout_selftest_kernel(int tag) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const AbortFlag abort{&abort_word};
  if (threadIdx.x == 0) mbar_wait(&bar, 0, abort, 99, tag);
  __syncthreads();
}
constexpr unsigned int kSelftestPolls = 1u << 12, kProductionPolls = 1u << 20;
// the poll limit travels on the stream, in front of and behind the self-test launch (pageable source: staged
// before the call returns)
int set_spin_limit_on(cudaStream_t stream, unsigned int polls) {
  return int(cudaMemcpyToSymbolAsync(g_spin_limit, &polls, sizeof(polls), 0, cudaMemcpyHostToDevice, stream));
}
}  // namespace

GDN_SM100_DEFINE_STATUS_HOOKS(umma)

int launch_wait_timeout_selftest(int tag, cudaStream_t stream) {
  if (int rc = set_spin_limit_on(stream, kSelftestPolls)) return rc;
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(tag);
  const int launched = int(cudaGetLastError());
  const int restored = set_spin_limit_on(stream, kProductionPolls);
  return launched ? launched : restored;
}

// The chunk walk with a producer that stops feeding it after the first chunk: every role of the real kernel runs
// out of its bounded wait (or sees the CTA-wide flag), the CTA drains, frees its tensor memory and returns.
int launch_walk_stall_selftest(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  if (int rc = set_spin_limit_on(stream, kSelftestPolls)) return rc;
  Inputs stalled = in;
  stalled.walk_flags = kWalkSelftestStall;
  Geometry one = geo;
  one.parallel = 0;
  const int launched = launch_walk_umma(stalled, one, ws, stream);
  const int restored = set_spin_limit_on(stream, kProductionPolls);
  return launched ? launched : restored;
}

int read_walk_plan_counts(int* host_out2, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out2, g_walk_plan_counts, 2 * sizeof(int));
  if (e != cudaSuccess) return int(e);
  if (reset) {
    const int zero[2] = {0, 0};
    e = cudaMemcpyToSymbol(g_walk_plan_counts, zero, sizeof(zero));
  }
  return int(e);
}

int read_device_status(int* host_out4, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out4, g_device_status, 4 * sizeof(int));
  if (e != cudaSuccess) return int(e);
  if (reset) {
    const int zero[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero));
  }
  return int(e);
}

}  // namespace gdn_sm100
