// out_proj of the layer's output gate: C[M,N] = A[M,K] W[N,K]^T, BF16 operands, FP32 accumulation, BF16 result
// (the reference's out_proj_gemm / out_proj_gemm_cutlass, csrc/output_gate/output_gate.cu and
// csrc/output_gate/output_gate_cutlass.cu, docs/OUTPUT_GATE.md:17-24: an mma.sync kernel and a CUTLASS SM80 GEMM).
// Here: one tcgen05 kernel.  A CTA owns a 128 x 128 tile of C; both operands are K-major as they lie in memory
// (A row-major, W in the Linear layout [N][K]), so their 128 x 64 tiles come straight from TMA into
// 128-byte-swizzled shared memory, three stages deep; the accumulator lives in 128 columns of tensor memory.
// Roles: warp 0 TMA producer, warp 1 MMA issuer (owns the tensor-memory allocation), warps 2-5 epilogue
// (TMEM -> registers -> BF16 -> 256 contiguous bytes per row and thread).  Two CTAs per SM, so the epilogue of one
// tile overlaps the main loop of another.  Rows and columns beyond M, N and the K tail read as zeros (TMA fill).
#include "actlize_la_sm100.h"
#include "gdn_common.cuh"
#include "umma.cuh"

namespace gdn_sm100 {
using namespace ptx;
namespace {

constexpr int kTileM = 128, kTileN = 128, kTileK = 64, kGemmStages = 3;
constexpr int kOperandBytes = kTileM * kTileK * 2;                 // 16 KB per operand tile
constexpr int kGemmStageBytes = 2 * kOperandBytes;
constexpr int kGemmBars = kGemmStages * kGemmStageBytes;
constexpr int kGemmSmem = kGemmBars + 128 + 1024;
constexpr int kGemmThreads = 192;
constexpr uint32_t kIdescGemm = idesc_bf16(kTileM, kTileN, false, false);
static_assert(2 * (kGemmSmem + 1024) <= 227 * 1024, "two GEMM CTAs must fit in one SM's shared memory");

__global__ void __launch_bounds__(kGemmThreads, 2)
out_proj_umma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                     __nv_bfloat16* __restrict__ c, int m, int n, int k) {
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* sm = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + kGemmBars);       // [stages] tiles landed
  uint64_t* empty = full + kGemmStages;                               // [stages] tiles consumed
  uint64_t* done = empty + kGemmStages;                               // accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const AbortFlag abort{abort_word};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN, m0 = blockIdx.y * kTileM;
  const int k_tiles = (k + kTileK - 1) / kTileK;

  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(done, 1);
    *abort_word = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTileN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&tm_a);
      prefetch_tensormap(&tm_w);
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % kGemmStages;
        if (kt >= kGemmStages && !mbar_wait(empty + s, ((kt / kGemmStages) - 1) & 1, abort, 60, kt)) break;
        uint8_t* stage = sm + s * kGemmStageBytes;
        mbar_arrive_expect_tx(full + s, kGemmStageBytes);
        tma_load_2d(stage, &tm_a, full + s, kt * kTileK, m0);
        tma_load_2d(stage + kOperandBytes, &tm_w, full + s, kt * kTileK, n0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t base = smem_u32(sm);
      bool ok = true;
      for (int kt = 0; kt < k_tiles && ok; ++kt) {
        const int s = kt % kGemmStages;
        ok = mbar_wait(full + s, (kt / kGemmStages) & 1, abort, 61, kt);
        tc_fence_after();
        const uint64_t da = smem_desc(base + s * kGemmStageBytes, 16, 1024);
        const uint64_t db = smem_desc(base + s * kGemmStageBytes + kOperandBytes, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < kTileK / 16; ++ks)          // 16 BF16 (32 bytes) along K per instruction
          mma_ss(tmem, da + uint64_t(ks * 2), db + uint64_t(ks * 2), kIdescGemm, (kt | ks) != 0);
        mma_commit(empty + s);
      }
      mma_commit(done);
    }
    __syncwarp();
  } else {
    // epilogue: a warp may only touch the TMEM lane quarter (warp % 4); warps 2..5 cover quarters 2, 3, 0, 1
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    const bool ok = mbar_wait(done, 0, abort, 62, 0);
    tc_fence_after();
    if (ok) {
      const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16);
#pragma unroll
      for (int piece = 0; piece < kTileN / 32; ++piece) {
        uint32_t d[32];
        tmem_ld32(taddr + piece * 32, d);        // warp-collective: every lane takes part, also rows beyond M
        tmem_wait_ld();
        if (row < m) {
          __nv_bfloat16* dst = c + (long long)row * n + n0 + piece * 32;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (n0 + piece * 32 + q * 8 < n) {     // N is a multiple of 8: a 16-byte piece is inside or outside
              uint4 o;
              o.x = pack_bf16(__uint_as_float(d[q * 8 + 0]), __uint_as_float(d[q * 8 + 1]));
              o.y = pack_bf16(__uint_as_float(d[q * 8 + 2]), __uint_as_float(d[q * 8 + 3]));
              o.z = pack_bf16(__uint_as_float(d[q * 8 + 4]), __uint_as_float(d[q * 8 + 5]));
              o.w = pack_bf16(__uint_as_float(d[q * 8 + 6]), __uint_as_float(d[q * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + q * 8) = o;
            }
          }
        }
      }
    }
  }
  if (abort.raised()) {
    for (int i = 0; i < 20; ++i) __nanosleep(100000);   // let copies in flight land before the CTA leaves
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTileN);
}

}  // namespace

GDN_SM100_DEFINE_STATUS_HOOKS(gemm)

int configure_out_proj() {
  if (int rc = tensor_map_encoder().init()) return rc;
  return int(cudaFuncSetAttribute(out_proj_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem));
}

int launch_out_proj(const void* a, const void* w, void* c, int m, int n, int k, cudaStream_t stream) {
  TensorMapEncoder& enc = tensor_map_encoder();
  if (int rc = enc.init()) return rc;
  CUtensorMap tm_a, tm_w;
  if (int rc = enc.bf16_2d(&tm_a, a, uint64_t(k), uint64_t(m), kTileM)) return rc;
  if (int rc = enc.bf16_2d(&tm_w, w, uint64_t(k), uint64_t(n), kTileN)) return rc;
  const dim3 grid((n + kTileN - 1) / kTileN, (m + kTileM - 1) / kTileM);
  out_proj_umma_kernel<<<grid, kGemmThreads, kGemmSmem, stream>>>(tm_a, tm_w, static_cast<__nv_bfloat16*>(c), m, n, k);
  return int(cudaGetLastError());
}

}  // namespace gdn_sm100

using namespace gdn_sm100;

extern "C" int actlize_la_sm100_out_proj(const void* a, const void* w, void* c, int m, int n, int k, void* stream) {
  if (!a || !w || !c || m <= 0 || n <= 0 || k <= 0) return int(cudaErrorInvalidValue);
  if ((n & 7) || (k & 7)) return int(cudaErrorInvalidValue);               // 16-byte rows for TMA and the stores
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(c) & 15))
    return int(cudaErrorInvalidValue);
  if ((m + kTileM - 1) / kTileM > 65535) return int(cudaErrorInvalidValue);
  return launch_out_proj(a, w, c, m, n, k, static_cast<cudaStream_t>(stream));
}
