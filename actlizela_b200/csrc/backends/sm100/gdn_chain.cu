// Chained chunk walk (configuration "chain") for sm_100a.
//
// The plain tensor-core walk forms N_c = U_c - W_c S_c only after the state S_c is complete and has been split
// into BF16 operands, so one chunk costs  split -> W S -> N -> state update  in series.  Here the product is
// expanded one step:
//     S_c     = gamma_{c-1} S_{c-1} + K_{c-1}^T (N*rel)_{c-1}
//     W_c S_c = (gamma_{c-1} W_c) S_{c-1} + (W_c K_{c-1}^T) (N*rel)_{c-1}  =  W~_c S_{c-1} + G_c (N*rel)_{c-1}
// W~ (W scaled by the previous chunk's decay) and G (64 x 64) come from the prepare stage.  The first term
// only needs the split of S_{c-1}, which is done while chunk c-1 is still being processed; the second term is
// 8 short instructions issued as soon as (N*rel)_{c-1} exists.  The serial chain per chunk shrinks to
//     N operands written -> G (N*rel) -> N of the next chunk,
// and the state update and its split run beside it on their own warps.  The first chunk of a launch has
// W~ = W and no G term.  Math reference: the WY chunk form of the reference project (tests/wy_cpu.py:44-88).
//
// Orientation, precision and operand formats are those of the plain tensor-core walk (gdn_umma.cu): state
// transposed St[v][k] in tensor memory, M = 128 value rows, BF16 hi/lo operands on the state path.
#include "gdn_common.cuh"
#include "umma.cuh"
#include <type_traits>

namespace gdn_sm100 {
using namespace ptx;
namespace {

constexpr int kBox = 8192;   // one TMA box: 64 rows x 128 bytes
constexpr uint32_t kIdescN64 = idesc_bf16(128, 64, false, false);
constexpr uint32_t kIdescN128 = idesc_bf16(128, 128, false, false);
constexpr uint32_t kIdescN128BT = idesc_bf16(128, 128, false, true);   // B MN-major

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// One CTA per (batch, value head), 768 threads, one CTA per SM.  Tensor memory (512 columns):
//   ACC_S [  0,128)  St FP32 accumulator (holds gamma_c * St once chunk c has been split)
//   OP_SH [128,192)  St BF16 hi, packed pairs      OP_SL [192,256)  St BF16 lo
//   ACC_Z [256,384)  [ (W~_hi S + G_hi NR + W~_hi S_lo + G_hi NR_lo)^T | (W~_lo S + G_lo NR)^T ]
//   ACC_O [384,448)  O^T = St Qs^T + N^T P^T
//   OP_NR [448,512)  per 16-token group ks: (N*rel) hi at 16ks, lo at 16ks+8 (packed pairs)
// N itself (BF16, for P N) goes through a shared-memory tile because tensor memory is full.
// The split of S_c feeds two products, Z_{c+1} and the state part of O_c; they are one 192-column instruction
// stream with B = [W~_hi ; W~_lo](c+1) stacked on Qs(c), which is why ring A pairs W~ of a chunk with the
// scaled queries of the chunk before it.
// Shared memory: ring A (two stages): per 64-wide key atom [W~_hi | W~_lo](c) [Qs](c-1), then [G_hi | G_lo](c);
// ring B (two stages): K, P, gate vector of chunk c.
// Roles: warps 0 and 2 MMA issuers, warp 1 TMA producer, warps 4-11 N step (quarter = warp & 3 owns 32 TMEM lanes,
// half = token half), warps 12-19 state split (half = key-column half), warps 20-23 output.
struct ChainLayout {
  static constexpr int kW0 = 0, kW1 = 3 * kBox, kQs = 2 * kBox, kG = 6 * kBox;    // kQs: offset inside an atom
  static constexpr int kStageA = 8 * kBox, kTxA = 8 * kBox;
  static constexpr int kK = 0, kP = 2 * kBox, kGates = 3 * kBox;
  static constexpr int kStageB = 3 * kBox + 1024, kTxB = 3 * kBox + 512;
  static constexpr int kRingA = 0, kRingB = 2 * kStageA;
  static constexpr int kN16 = kRingB + 2 * kStageB;     // [128 value rows][64 tokens] BF16, 128-byte swizzle
  static constexpr int kOut = kN16 + 2 * kBox;          // one staging tile [64 tokens][128 values] BF16
  static constexpr int kBars = kOut + 2 * kBox;
  static constexpr int kTotal = kBars + 256;
};
constexpr int kMmaWarp = 0, kTmaWarp = 1, kMmaWarp2 = 2, kNWarp0 = 4, kSplitWarp0 = 12, kOutWarp0 = 20;
constexpr int kChainThreads = 768;
constexpr int kChainSmem = ChainLayout::kTotal + 1024;
static_assert(kChainSmem <= 232448, "shared memory of one CTA");
constexpr uint32_t kAccS = 0, kOpSH = 128, kOpSL = 192, kAccZ = 256, kAccO = 384, kOpNR = 448;
constexpr uint32_t kIdescN192 = idesc_bf16(128, 192, false, false);

// Diagnostic build: clock stamps (cycles since kernel start) into the unused tail of the chunk's gate vector.
#ifdef GDN_SM100_PHASE_TIMING
#define GDN_CSTAMP(leader_tid, chunk, slot) \
  if (tid == (leader_tid)) ws.gates[(block0 + (chunk)) * 128 + 96 + (slot)] = float((clock64() - t_begin) & 0xffffff)
#else
#define GDN_CSTAMP(leader_tid, chunk, slot)
#endif

__global__ void __launch_bounds__(kChainThreads, 1)
walk_chain_kernel(const __grid_constant__ CUtensorMap tm_wh, const __grid_constant__ CUtensorMap tm_wl,
                  const __grid_constant__ CUtensorMap tm_gh, const __grid_constant__ CUtensorMap tm_gl,
                  const __grid_constant__ CUtensorMap tm_qs, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_out,
                  Inputs in, Geometry geo, Workspace ws) {
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* sm = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  using L = ChainLayout;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L::kBars);
  uint64_t* full_a = bars;            // [2]
  uint64_t* empty_a = bars + 2;       // [2]
  uint64_t* full_b = bars + 4;        // [2]
  uint64_t* empty_b = bars + 6;       // [2]
  uint64_t* bar_ops = bars + 8;       // [2] state operands written, first / second K half (one arrival per split warp)
  uint64_t* bar_opn = bars + 10;      // [2] N operands written, token groups {0,2} / {1,3} (one arrival per N warp)
  uint64_t* bar_z = bars + 12;        // W S accumulator complete
  uint64_t* bar_zread = bars + 13;    // W S accumulator has been read (one arrival per N warp)
  uint64_t* bar_s = bars + 14;        // state update complete
  uint64_t* bar_o = bars + 15;        // output accumulator complete
  uint64_t* bar_ofree = bars + 16;    // output accumulator drained (one arrival per output warp)
  uint64_t* bar_staged = bars + 17;   // output tile staged (one arrival per output warp)
  uint64_t* bar_stfree = bars + 18;   // staging tile read out by its store
  uint64_t* bar_xq = bars + 19;       // products fed by a split complete (second issuer -> first issuer, split warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const AbortFlag abort{abort_word};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x;
  const int b = bh / geo.value_heads, hv = bh % geo.value_heads;
  const int hk = hv / geo.group();
  const int chunks = geo.segment_chunks(), c0 = geo.chunk_begin;     // this launch walks chunks [c0, c0 + chunks)
  const long long block0 = (long long)bh * geo.chunks() + c0;
  const float* state_in = geo.first_segment() ? in.initial : ws.carry;
  float* state_out = geo.last_segment() ? in.final_state : ws.carry;
#ifdef GDN_SM100_PHASE_TIMING
  const long long t_begin = clock64();
#endif

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(full_a + s, 1);
      mbar_init(empty_a + s, 1);
      mbar_init(full_b + s, 1);
      mbar_init(empty_b + s, 1);
      mbar_init(bar_ops + s, 8);
      mbar_init(bar_opn + s, 8);
    }
    mbar_init(bar_z, 1);
    mbar_init(bar_zread, 8);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_init(bar_ofree, 4);
    mbar_init(bar_staged, 4);
    mbar_init(bar_stfree, 1);
    mbar_init(bar_xq, 1);
    *abort_word = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= kNWarp0 && warp < kSplitWarp0) {
    // ------------------------------------------------------------------ N step: N = U - Z, operands for the MMAs
    const int quarter = warp & 3, half = (warp - kNWarp0) >> 2;
    const int v = quarter * 32 + lane;                     // value row = TMEM lane
    const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16);
    uint8_t* n16row = sm + L::kN16 + (v >> 3) * 1024 + (v & 7) * 128;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int s = c & 1;
      const float* gates = reinterpret_cast<const float*>(sm + L::kRingB + s * L::kStageB + L::kGates);
      const float* urow = ws.u + ((block0 + c) * kChunk + half * 32) * kDim + v;
      if (c + 1 < chunks)      // pull the next chunk's U rows of this warp towards L2
        asm volatile("prefetch.global.L2 [%0];" ::"l"(urow + kChunk * kDim + lane * kDim - lane));
      float u[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) u[i] = __ldg(urow + i * kDim);
      ok = mbar_wait(full_b + s, (c >> 1) & 1, abort, 11, c);
      ok = ok && mbar_wait(bar_z, c & 1, abort, 12, c);
      if (!ok) break;
      tc_fence_after();
      GDN_CSTAMP(kNWarp0 * 32, c, 2);
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int ks = half * 2 + part;                     // 16-token group
        uint32_t nh[8], nl[8], n16[8];
        {
          uint32_t dh[16], dl[16];
          tmem_ld16(taddr + kAccZ + ks * 16, dh);
          tmem_ld16(taddr + kAccZ + 64 + ks * 16, dl);
          tmem_wait_ld();
          if (part == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_zread);
          }
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const int i = ks * 16 + j;
            const float n0 = u[part * 16 + j] - (__uint_as_float(dh[j]) + __uint_as_float(dl[j]));
            const float n1 = u[part * 16 + j + 1] - (__uint_as_float(dh[j + 1]) + __uint_as_float(dl[j + 1]));
            const float r0 = n0 * gates[i], r1 = n1 * gates[i + 1];
            const uint32_t h = pack_bf16(r0, r1);
            nh[j >> 1] = h;
            nl[j >> 1] = pack_bf16(r0 - bf16_lo(h), r1 - bf16_hi(h));
            n16[j >> 1] = pack_bf16(n0, n1);
          }
        }
        // (the previous chunk's N operands and N tile are free: the commit that completed bar_z was issued
        // behind every instruction that reads them)
        tmem_st8(taddr + kOpNR + ks * 16, nh);
        tmem_st8(taddr + kOpNR + ks * 16 + 8, nl);
        *reinterpret_cast<uint4*>(n16row + (((2 * ks) ^ (v & 7)) << 4)) = make_uint4(n16[0], n16[1], n16[2], n16[3]);
        *reinterpret_cast<uint4*>(n16row + (((2 * ks + 1) ^ (v & 7)) << 4)) = make_uint4(n16[4], n16[5], n16[6], n16[7]);
        tmem_wait_st();
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_opn + part);
      }
      GDN_CSTAMP(kNWarp0 * 32, c, 4);
    }
  } else if (warp >= kSplitWarp0 && warp < kOutWarp0) {
    // ------------------------------------------------------------------ state split (and state in / out)
    const int quarter = warp & 3, half = (warp - kSplitWarp0) >> 2;
    const int v = quarter * 32 + lane;
    const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16);
    {
      const float* init = state_in ? state_in + (long long)bh * kDim * kDim + v : nullptr;
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        uint32_t vals[16];
        const int k0 = half * 64 + part * 16;
#pragma unroll
        for (int j = 0; j < 16; ++j) vals[j] = init ? __float_as_uint(init[(k0 + j) * kDim]) : 0u;
        tmem_st16(taddr + kAccS + k0, vals);
      }
      tmem_wait_st();
    }
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int s = c & 1;
      const float* gates = reinterpret_cast<const float*>(sm + L::kRingB + s * L::kStageB + L::kGates);
      // S_c is complete; the products that read the previous split were issued before that update
      // ... by the other issuer: wait for them too before the operands are replaced
      if (c > 0) ok = mbar_wait(bar_s, (c - 1) & 1, abort, 10, c) && mbar_wait(bar_xq, (c - 1) & 1, abort, 16, c);
      ok = ok && mbar_wait(full_b + s, (c >> 1) & 1, abort, 14, c);
      if (!ok) break;
      tc_fence_after();
      GDN_CSTAMP(kSplitWarp0 * 32, c, 0);
      const float gamma = gates[kChunk];
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        uint32_t d[16], hi[8], lo[8];
        const int k0 = half * 64 + part * 16;
        tmem_ld16(taddr + kAccS + k0, d);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float s0 = __uint_as_float(d[j]), s1 = __uint_as_float(d[j + 1]);
          const uint32_t h = pack_bf16(s0, s1);
          hi[j >> 1] = h;
          lo[j >> 1] = pack_bf16(s0 - bf16_lo(h), s1 - bf16_hi(h));
          d[j] = __float_as_uint(s0 * gamma);
          d[j + 1] = __float_as_uint(s1 * gamma);
        }
        tmem_st8(taddr + kOpSH + (k0 >> 1), hi);
        tmem_st8(taddr + kOpSL + (k0 >> 1), lo);
        tmem_st16(taddr + kAccS + k0, d);
        if (part & 1) {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_ops + (part >> 1));
        }
      }
      GDN_CSTAMP(kSplitWarp0 * 32, c, 1);
    }
    if (ok) ok = mbar_wait(bar_s, (chunks - 1) & 1, abort, 15, chunks);
    if (ok && state_out) {
      tc_fence_after();
      float* fin = state_out + (long long)bh * kDim * kDim + v;
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        uint32_t d[16];
        const int k0 = half * 64 + part * 16;
        tmem_ld16(taddr + kAccS + k0, d);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) fin[(k0 + j) * kDim] = __uint_as_float(d[j]);
      }
    }
  } else if (warp >= kOutWarp0) {
    // ------------------------------------------------------------------ output epilogue
    const int quarter = warp - kOutWarp0;
    const int v = quarter * 32 + lane;
    const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16) + kAccO;
    uint8_t* stage = sm + L::kOut + (v >> 6) * kBox + ((v & 7) << 1);
    const int chunk16 = (v & 63) >> 3;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      ok = mbar_wait(bar_o, c & 1, abort, 20, c);
      if (!ok) break;
      tc_fence_after();
      GDN_CSTAMP(kOutWarp0 * 32, c, 5);
      uint32_t o0[32], o1[32];
      tmem_ld32(taddr, o0);
      tmem_ld32(taddr + 32, o1);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ofree);
      // the previous chunk's store must have read the staging tile before it is rewritten
      if (c > 0) ok = mbar_wait(bar_stfree, (c - 1) & 1, abort, 21, c);
      if (!ok) break;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        *reinterpret_cast<__nv_bfloat16*>(stage + i * 128 + ((chunk16 ^ (i & 7)) << 4)) =
            __float2bfloat16_rn(__uint_as_float(o0[i]));
#pragma unroll
      for (int i = 0; i < 32; ++i)
        *reinterpret_cast<__nv_bfloat16*>(stage + (32 + i) * 128 + ((chunk16 ^ (i & 7)) << 4)) =
            __float2bfloat16_rn(__uint_as_float(o1[i]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_staged);
      if (tid == kOutWarp0 * 32) {
        ok = mbar_wait(bar_staged, c & 1, abort, 22, c);
        if (!ok) break;
        const uint8_t* tile = sm + L::kOut;
        tma_store_4d(&tm_out, tile, 0, hv, (c0 + c) * kChunk, b);
        tma_store_4d(&tm_out, tile + kBox, 64, hv, (c0 + c) * kChunk, b);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(bar_stfree);
      }
    }
    if (tid == kOutWarp0 * 32) tma_store_wait_all();
  } else if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_wh);
      prefetch_tensormap(&tm_wl);
      prefetch_tensormap(&tm_gh);
      prefetch_tensormap(&tm_gl);
      prefetch_tensormap(&tm_qs);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_p);
      // ring A has one more fill than there are chunks: the last one only carries the last chunk's queries
      for (int c = 0; c <= chunks; ++c) {
        const int s = c & 1;
        const int row = int((block0 + c) * kChunk);
        if (c >= 2 && !mbar_wait(empty_a + s, ((c >> 1) - 1) & 1, abort, 30, c)) break;
        uint8_t* sa = sm + L::kRingA + s * L::kStageA;
        mbar_arrive_expect_tx(full_a + s, c < chunks ? L::kTxA : 2 * kBox);
        tma_load_2d(sa + L::kW0 + L::kQs, &tm_qs, full_a + s, 0, row - kChunk);      // row -64 of the first block: zero fill
        tma_load_2d(sa + L::kW1 + L::kQs, &tm_qs, full_a + s, 64, row - kChunk);
        if (c == chunks) break;
        tma_load_2d(sa + L::kW0, &tm_wh, full_a + s, 0, row);
        tma_load_2d(sa + L::kW0 + kBox, &tm_wl, full_a + s, 0, row);
        tma_load_2d(sa + L::kW1, &tm_wh, full_a + s, 64, row);
        tma_load_2d(sa + L::kW1 + kBox, &tm_wl, full_a + s, 64, row);
        tma_load_2d(sa + L::kG, &tm_gh, full_a + s, 0, row);
        tma_load_2d(sa + L::kG + kBox, &tm_gl, full_a + s, 0, row);
        if (c >= 2 && !mbar_wait(empty_b + s, ((c >> 1) - 1) & 1, abort, 31, c)) break;
        uint8_t* sb = sm + L::kRingB + s * L::kStageB;
        mbar_arrive_expect_tx(full_b + s, L::kTxB);
        bulk_load(sb + L::kGates, ws.gates + (block0 + c) * 128, 512, full_b + s);
        tma_load_4d(sb + L::kK, &tm_k, full_b + s, 0, hk, (c0 + c) * kChunk, b);
        tma_load_4d(sb + L::kK + kBox, &tm_k, full_b + s, 64, hk, (c0 + c) * kChunk, b);
        tma_load_2d(sb + L::kP, &tm_p, full_b + s, 0, row);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp || warp == kMmaWarp2) {
    // ------------------------------------------------------------------ MMA issuers
    // One thread cannot issue a chunk's 36 instructions and poll a dozen barriers fast enough, so the work is
    // divided by what it waits for: warp 0 follows the N operands (state update, G term, P N), warp 2 follows the
    // state split (the 192-column product).  tcgen05.mma of different threads are ordered only through
    // commit -> mbarrier -> wait -> fence, which is what bar_xq / bar_z / bar_s / bar_o provide.
    // The issuing threads are latency-bound scalar programs: the steady-state loops below are peeled so that they
    // hold no data-dependent branch but one check of the wait results per chunk (a wait that gave up lets the
    // rest of that chunk's instructions run on stale operands, which is harmless: the launch is already failed),
    // and the base addresses are broadcast so that the compiler knows they are warp-uniform.
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t base = __shfl_sync(0xffffffffu, smem_u32(sm), 0);
    if (lane == 0) {
      bool ok = true;
      // Descriptors of ring stage 0; stage 1 is a constant further on (the start-address field counts 16-byte units).
      const uint64_t dN16 = smem_desc(base + L::kN16, 16, 1024);
      const uint64_t dW0s = smem_desc(base + L::kRingA + L::kW0, 16, 1024);
      const uint64_t dW1s = smem_desc(base + L::kRingA + L::kW1, 16, 1024);
      const uint64_t dGs = smem_desc(base + L::kRingA + L::kG, 16, 1024);
      const uint64_t dKs = smem_desc(base + L::kRingB + L::kK, kBox, 1024);
      const uint64_t dPs = smem_desc(base + L::kRingB + L::kP, 16, 1024);
      auto in_a = [](uint64_t d, int s) { return d + uint64_t(s * (L::kStageA >> 4)); };
      auto in_b = [](uint64_t d, int s) { return d + uint64_t(s * (L::kStageB >> 4)); };
      if (warp == kMmaWarp2) {
        // One half of the products fed by the split of S_{j-1} (ring A stage of chunk j):
        //   [Z_j | O_{j-1}] = SH [W~_hi ; W~_lo ; Qs]^T,  Z_j[0,64) += SL W~_hi^T.
        // kMode 0: both (192 columns), 1: Z only (chunk 0: there is no chunk before it), 2: O only (behind the
        // last chunk).  K steps {0,1,4,5} of the split become available first (part 0), {2,3,6,7} second.
        auto split_products = [&](int s, int part, auto mode) {
          constexpr int kMode = decltype(mode)::value;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int ks = (q >> 1) * 4 + part * 2 + (q & 1);
            const uint64_t bdesc = in_a((ks >> 2) ? dW1s : dW0s, s) + uint64_t((ks & 3) * 2);   // +32 bytes per K step
            const uint32_t acc = (part | q) != 0;
            if (kMode == 0) mma_ts(tm + kAccZ, tm + kOpSH + ks * 8, bdesc, kIdescN192, acc);
            if (kMode == 1) mma_ts(tm + kAccZ, tm + kOpSH + ks * 8, bdesc, kIdescN128, acc);
            if (kMode == 2) mma_ts(tm + kAccO, tm + kOpSH + ks * 8, bdesc + uint64_t(L::kQs >> 4), kIdescN64, acc);
            if (kMode != 2) mma_ts(tm + kAccZ, tm + kOpSL + ks * 8, bdesc, kIdescN64, 1);
          }
        };
        using Both = std::integral_constant<int, 0>;
        using OnlyZ = std::integral_constant<int, 1>;
        using OnlyO = std::integral_constant<int, 2>;
        // split of the incoming state -> Z_0 (complete as it is: there is no G term) ...
        ok = mbar_wait(full_a, 0, abort, 40, 0) & mbar_wait(bar_ops, 0, abort, 41, 0);
        tc_fence_after();
        split_products(0, 0, OnlyZ{});
        ok &= mbar_wait(bar_ops + 1, 0, abort, 41, 0);
        tc_fence_after();
        split_products(0, 1, OnlyZ{});
        mma_commit(bar_z);
        mma_commit(empty_a);
        // ... and, if there is a second chunk, [Z_1 | O_0]
        if (chunks > 1) {
          ok &= mbar_wait(full_a + 1, 0, abort, 40, 1) & mbar_wait(bar_zread, 0, abort, 44, 1);
          tc_fence_after();
          split_products(1, 0, Both{});
          split_products(1, 1, Both{});
          mma_commit(bar_xq);
        }
        // split of S_j -> [Z_{j+1} | O_j], ring A stage of chunk j+1
        for (int j = 1; j + 1 < chunks && ok; ++j) {
          const int sn = (j + 1) & 1;
          ok = mbar_wait(full_a + sn, ((j + 1) >> 1) & 1, abort, 40, j + 1) &
               mbar_wait(bar_ofree, (j - 1) & 1, abort, 45, j) & mbar_wait(bar_zread, j & 1, abort, 44, j + 1) &
               mbar_wait(bar_ops, j & 1, abort, 41, j);
          tc_fence_after();
          split_products(sn, 0, Both{});
          ok &= mbar_wait(bar_ops + 1, j & 1, abort, 41, j);
          tc_fence_after();
          split_products(sn, 1, Both{});
          mma_commit(bar_xq);
        }
        // split of the last chunk's state: only the state part of its output is left
        if (ok) {
          const int j = chunks - 1, sn = (j + 1) & 1;
          ok = mbar_wait(full_a + sn, ((j + 1) >> 1) & 1, abort, 40, j + 1);
          if (j > 0)
            ok &= mbar_wait(bar_ofree, (j - 1) & 1, abort, 45, j) & mbar_wait(bar_ops, j & 1, abort, 41, j) &
                  mbar_wait(bar_ops + 1, j & 1, abort, 41, j);
          tc_fence_after();
          split_products(sn, 0, OnlyO{});
          split_products(sn, 1, OnlyO{});
          mma_commit(bar_xq);
        }
      } else {
        // state update  St += (N*rel)^T K  (the accumulator already holds gamma_j St) for one token half
        auto update_part = [&](int s, int part) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int ks = h * 2 + part;
            const uint64_t kdesc = in_b(dKs, s) + uint64_t(ks * 128);                           // +2048 bytes per K step
            mma_ts(tm + kAccS, tm + kOpNR + ks * 16, kdesc, kIdescN128BT, 1);
            mma_ts(tm + kAccS, tm + kOpNR + ks * 16 + 8, kdesc, kIdescN128BT, 1);
          }
        };
        // Z_{j+1} += (N*rel)_j^T [G_hi ; G_lo]^T, low part of N*rel only against G_hi
        auto g_part = [&](int sn, int part) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int ks = h * 2 + part;
            const uint64_t gdesc = in_a(dGs, sn) + uint64_t(ks * 2);
            mma_ts(tm + kAccZ, tm + kOpNR + ks * 16, gdesc, kIdescN128, 1);
            mma_ts(tm + kAccZ, tm + kOpNR + ks * 16 + 8, gdesc, kIdescN64, 1);
          }
        };
        // O_j^T += N^T P^T (N from the shared-memory tile)
        auto output_product = [&](int s) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tm + kAccO, dN16 + uint64_t(ks * 2), in_b(dPs, s) + uint64_t(ks * 2), kIdescN64, 1);
        };
        int j = 0;
        for (; j + 1 < chunks && ok; ++j) {
          const int s = j & 1, sn = s ^ 1;
          // N operands of the first token half; K of this chunk; the split has scaled the accumulator by gamma_j
          ok = mbar_wait(bar_opn, j & 1, abort, 43, j) & mbar_wait(full_b + s, (j >> 1) & 1, abort, 42, j) &
               mbar_wait(bar_ops + 1, j & 1, abort, 46, j);
          tc_fence_after();
          update_part(s, 0);           // first: the split of the new state waits for it
          // the other issuer's product [Z_{j+1} | O_j] must be complete before anything is added to it
          ok &= mbar_wait(bar_xq, j & 1, abort, 47, j) & mbar_wait(full_a + sn, ((j + 1) >> 1) & 1, abort, 40, j + 1);
          tc_fence_after();
          g_part(sn, 0);
          ok &= mbar_wait(bar_opn + 1, j & 1, abort, 43, j);
          tc_fence_after();
          update_part(s, 1);
          mma_commit(bar_s);
          // P N goes in front of the last G instructions: the commit behind those then tells the N warps both that
          // Z_{j+1} is complete and that every reader of this chunk's N operands is done
          output_product(s);
          mma_commit(bar_o);
          mma_commit(empty_b + s);
          g_part(sn, 1);
          mma_commit(bar_z);
          mma_commit(empty_a + sn);
        }
        if (ok) {      // last chunk: no next Z
          const int s = j & 1;
          ok = mbar_wait(bar_opn, j & 1, abort, 43, j) & mbar_wait(full_b + s, (j >> 1) & 1, abort, 42, j) &
               mbar_wait(bar_ops + 1, j & 1, abort, 46, j);
          tc_fence_after();
          update_part(s, 0);
          ok &= mbar_wait(bar_opn + 1, j & 1, abort, 43, j);
          tc_fence_after();
          update_part(s, 1);
          mma_commit(bar_s);
          ok &= mbar_wait(bar_xq, j & 1, abort, 47, j);
          tc_fence_after();
          output_product(s);
          mma_commit(bar_o);
          mma_commit(empty_b + s);
        }
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

}  // namespace

GDN_SM100_DEFINE_STATUS_HOOKS(chain)

int configure_chain() {
  if (int rc = tensor_map_encoder().init()) return rc;
  return int(cudaFuncSetAttribute(walk_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmem));
}

int launch_walk_chain(const Inputs& in, const Geometry& geo, const Workspace& ws, cudaStream_t stream) {
  TensorMapEncoder& enc = tensor_map_encoder();
  if (int rc = enc.init()) return rc;
  const uint64_t rows = uint64_t(geo.blocks()) * kChunk;
  CUtensorMap tm_wh, tm_wl, tm_gh, tm_gl, tm_qs, tm_k, tm_p, tm_out;
  if (int rc = enc.bf16_4d(&tm_out, in.output, kDim, geo.value_heads, geo.sequence, geo.batch, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_wh, ws.w_hi, kDim, rows, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_wl, ws.w_lo, kDim, rows, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_gh, ws.g_hi, kChunk, rows, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_gl, ws.g_lo, kChunk, rows, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_qs, ws.qs, kDim, rows, kChunk)) return rc;
  if (int rc = enc.bf16_4d(&tm_k, in.k, kDim, geo.key_heads, geo.sequence, geo.batch, kChunk)) return rc;
  if (int rc = enc.bf16_2d(&tm_p, ws.p, kChunk, rows, kChunk)) return rc;
  walk_chain_kernel<<<geo.batch * geo.value_heads, kChainThreads, kChainSmem, stream>>>(
      tm_wh, tm_wl, tm_gh, tm_gl, tm_qs, tm_k, tm_p, tm_out, in, geo, ws);
  return int(cudaGetLastError());
}

}  // namespace gdn_sm100
