// Thin inline-PTX layer for the Blackwell (sm_100a) data path used by the tensor-core kernels:
// mbarrier, TMA (cp.async.bulk[.tensor], no multicast anywhere), tensor memory (tcgen05.alloc /
// ld / st) and the 5th-generation MMA (tcgen05.mma, operands from shared-memory descriptors or
// from tensor memory, accumulators in tensor memory).
//
// Every wait is bounded: a wait that exceeds its spin limit records where it gave up in a
// device status word, raises a CTA-wide abort flag and returns false; callers leave their
// loops, the CTA drains, frees its tensor memory and returns.  Nothing traps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace gdn_sm100 {

// Status word of the translation unit that includes this header (the tensor-core kernels live in
// one translation unit): [0] first failure code (0 = none), [1] block index, [2] wait site, [3] chunk.
static __device__ int g_device_status[4];
// Host-visible copy of the same record (pinned, mapped host memory; null until configure() has set it): written
// once by the CTA that records a failure, so the host can notice a launch that gave up without synchronising.
static __device__ int* g_status_mirror;
// Poll limit of every bounded wait; the failure-detection self-test lowers it for one launch.
static __device__ unsigned int g_spin_limit = 1u << 20;

namespace ptx {


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

struct AbortFlag {
  volatile int* flag;   // shared-memory word, 0 while healthy
  __device__ __forceinline__ bool raised() const { return *flag != 0; }
  __device__ __forceinline__ void raise(int code, int site, int chunk) const {
    *flag = code;
    if (atomicCAS(&g_device_status[0], 0, code) == 0) {
      g_device_status[1] = blockIdx.x;
      g_device_status[2] = site;
      g_device_status[3] = chunk;
      volatile int* mirror = g_status_mirror;
      if (mirror) {
        mirror[1] = blockIdx.x;
        mirror[2] = site;
        mirror[3] = chunk;
        __threadfence_system();
        mirror[0] = code;
      }
    }
  }
};

// Bounded wait for the phase with the given parity.  Returns false after a time-out or when
// another role of this CTA has already given up.
// The polling loop is one shared out-of-line routine: inlined at the ~40 wait sites of a warp-specialised kernel
// it made up a third of the kernel's code, and the issuing threads, which run their code alone, then paid an
// instruction-cache miss at nearly every wait.
static __device__ __noinline__ bool mbar_wait_poll(uint32_t bar_addr, uint32_t parity, volatile int* flag, int site,
                                            int chunk) {
  const AbortFlag abort{flag};
  const uint32_t limit = g_spin_limit;
  for (uint32_t spin = 0; spin < limit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 255u) == 255u && abort.raised()) return false;
  }
  abort.raise(1, site, chunk);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortFlag& abort,
                                          int site, int chunk) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_poll(smem_u32(bar), parity, abort.flag, site, chunk);
}

// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ TMA (never multicast)
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// plain bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// TMA store shared -> global of one box; the issuing thread later commits and waits on the group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed stores of this thread have finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// all but the most recent committed store group have finished reading shared memory
__device__ __forceinline__ void tma_store_wait_read_keep1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
// every committed store of this thread is complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------ tensor memory
// Allocation is warp-collective; the base address (lane 0, column c) is written to `slot`.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32-bit, 16 consecutive columns: thread i of the warp owns TMEM lane (base lane + i);
// v[j] is column (col + j).  `taddr` = (lane base << 16) | column.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// 32 consecutive columns per thread (same lane rule as above)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
               : "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor, 128-byte swizzle, tiles 1024-byte aligned.
//   K-major  operand: rows (M or N index) are 128-byte lines holding 64 BF16 along K; groups of 8 rows
//                     are `sbo` bytes apart (1024 when dense); `lbo` is unused (set to 16).
//   MN-major operand: 128-byte lines hold 64 BF16 along M/N; consecutive K indices are consecutive lines;
//                     groups of 8 K-lines are `sbo` bytes apart (1024 when dense); the next 64-wide M/N
//                     group is `lbo` bytes away.
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= 1ull << 46;    // descriptor version of this architecture
  d |= 2ull << 61;    // 128-byte swizzle
  return d;
}

// Instruction descriptor for kind::f16 with BF16 operands and FP32 accumulation.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                        // D format: F32
         | (1u << 7)                      // A format: BF16
         | (1u << 10)                     // B format: BF16
         | ((a_mn_major ? 1u : 0u) << 15) // A major-ness
         | ((b_mn_major ? 1u : 0u) << 16) // B major-ness
         | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is K-major in tensor memory (lane = row, BF16 pairs per column).
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

}  // namespace ptx

// ------------------------------------------------------------------ host side: tensor maps
struct TensorMapEncoder {
  using Fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                          const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                          CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  Fn encode = nullptr;
  int init();   // resolves cuTensorMapEncodeTiled through the runtime; returns a cudaError_t value
  // BF16 tensor, innermost dimension first; box rows are 128 bytes (64 BF16), 128-byte swizzle,
  // out-of-range elements read as zero.
  int bf16_2d(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint32_t box_rows) const;
  int bf16_4d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
              uint32_t box_rows_d2) const;
  // FP32 matrix, box = 32 columns (128 bytes) x box_rows, no swizzle (dense box in shared memory)
  int f32_2d(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint32_t box_rows) const;
};
TensorMapEncoder& tensor_map_encoder();

// Per translation unit (the status words above are file-local): point the kernels at the host-visible record,
// clear the device record, set the poll limit.  Each returns a cudaError_t value.
#define GDN_SM100_DEFINE_STATUS_HOOKS(suffix)                                                        \
  int set_status_mirror_##suffix(int* device_pointer) {                                              \
    return int(cudaMemcpyToSymbol(g_status_mirror, &device_pointer, sizeof(device_pointer)));        \
  }                                                                                                  \
  int clear_device_status_##suffix() {                                                               \
    const int zero[4] = {0, 0, 0, 0};                                                                \
    return int(cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero)));                             \
  }                                                                                                  \
  int set_spin_limit_##suffix(unsigned int polls) {                                                  \
    return int(cudaMemcpyToSymbol(g_spin_limit, &polls, sizeof(polls)));                             \
  }

}  // namespace gdn_sm100
