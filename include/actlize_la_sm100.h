/* C ABI of the B200 (sm_100a) chunked gated-delta-rule forward.
 *
 * This is the native boundary of the `cuda_sm100` backend.  It has the shape of the
 * reference project's plain-C launch interfaces for its WY/residual kernel families
 *   csrc/backends/ppu15/launch.h:6-17   (forward / target_arch / configure / forward_prepared)
 *   csrc/backends/ppu10/launch.h:5-14   (configure / core_route_v2 / forward_prepared)
 * and follows their conventions (csrc/backends/ppu10/launch.cu:51-84):
 *   - every function returns 0 on success and a non-zero cudaError_t value otherwise
 *     (cudaErrorInvalidValue for rejected arguments); nothing throws across the boundary;
 *   - `stream` is the caller's CUDA stream as an opaque pointer (for PyTorch callers,
 *     torch.cuda.current_stream().cuda_stream); the library never synchronises it;
 *   - all buffers are caller-owned device memory; inputs are read-only; output, final
 *     state and workspace are disjoint; strides are implied by contiguity;
 *   - forward_prepared allocates nothing and queries no device property, so it can be
 *     replayed inside a captured graph once `configure` has run on that device.
 *
 * Tensor contract (unchanged from the reference's gdn_forward, README.md:33-46):
 *   q, k      [B, T, Hk, 128] BF16          v, output [B, T, Hv, 128] BF16
 *   g         [B, T, Hv] natural-log decay, FP32 if gate_fp32 else BF16
 *   beta      [B, T, Hv] BF16               Hv % Hk == 0, chunk 64, query scale 1/sqrt(128) built in
 *   initial   [B, Hv, 128, 128] FP32, K-by-V order, may be NULL (zero state)
 *   final     [B, Hv, 128, 128] FP32, may be NULL (no export)
 */
#ifndef ACTLIZE_LA_SM100_H_
#define ACTLIZE_LA_SM100_H_

#ifdef __cplusplus
extern "C" {
#endif

#define ACTLIZE_LA_SM100_ABI_VERSION 1

/* Kernel configurations of the static shape table (see sm100_policy.json). */
#define ACTLIZE_LA_SM100_CONFIG_SIMT 0      /* FP32 CUDA-core kernels: diagnostic / cross-check */
#define ACTLIZE_LA_SM100_CONFIG_UMMA 1      /* tcgen05 + TMEM + TMA kernels */
/* ids 2 and 3 mix the stages (2: CUDA-core prepare + tcgen05 walk, 3: the reverse) for diagnosis.
 * OR-ing one of the following into `config` restricts forward_prepared to a single stage
 * (per-kernel timing; the walk-only form needs a workspace filled by an earlier call). */
#define ACTLIZE_LA_SM100_STAGE_PREPARE_ONLY 0x10
#define ACTLIZE_LA_SM100_STAGE_WALK_ONLY 0x20
/* Two modifiers of a walk-only call of configuration 1, used by the sequence-parallel scheme (several walks over
 * one prepared workspace): WALK_HOMOGENEOUS treats U as zero, which with the identity as initial state yields the
 * state-transition matrix of the segment; WALK_UNTIL_DECAYED stops every (batch, value head) walk at the first chunk
 * boundary where the decay accumulated since the segment start is below exp(-40), leaving later output rows
 * untouched (final_state must be NULL). */
#define ACTLIZE_LA_SM100_WALK_HOMOGENEOUS 0x40
#define ACTLIZE_LA_SM100_WALK_UNTIL_DECAYED 0x80
/* A third walk-only form of configuration 1, on its own (no other modifier, no sub-segments): the OFFSET pass.  Per
 * (batch, value head) only the shortest suffix of the sequence whose accumulated decay is below exp(-40) (all of its
 * tokens contractions) is walked, from a zero state; no output row is written (`output` must still be a valid
 * buffer) and `final_state` (required) receives the state the sequence ends in from a zero incoming state, which to
 * exp(-40) is what it ends in from any.  A head without such a suffix is walked whole: then the result is bit-equal
 * to the ordinary zero-state walk.  It gives a sequence-parallel rank its outgoing state after a few chunks of work. */
#define ACTLIZE_LA_SM100_WALK_OFFSET_SUFFIX 0x100000
/* The offset pass and the transition pass (WALK_HOMOGENEOUS from an identity state, which the kernel makes itself) in
 * ONE launch, two CTAs per (batch, value head); also a walk-only form of configuration 1 on its own.  `final_state`
 * (required) then points at a block [2][B][Hv][128][128]: the transition matrices M, then the offsets b, of
 * S_out = M S_in + b.  `initial` is not read; `output` must be a valid buffer the caller does not need (the transition
 * CTAs of a segment that does not decay write their rows there). */
#define ACTLIZE_LA_SM100_WALK_PAIR 0x200000

/* ABI version of this library; the loader refuses a mismatch.
 * Counterpart: ala_abi_version in csrc/serving/abi.h:67-82. */
int actlize_la_sm100_abi_version(void);

/* Architecture the device code was built for: always 100.
 * Replaces actlize_la_ppu15_target_arch (csrc/backends/ppu15/launch.h:11). */
int actlize_la_sm100_target_arch(void);

/* Identity string of the numerical contract, "wy-splitbf16-state-bf16-out-sm100-v1".
 * Counterpart of the pybind attribute math_contract checked by
 * actlize_la/gdn_sm90_interface.py:19-20. */
const char* actlize_la_sm100_numerical_contract(void);

/* One-time per-device set-up (shared-memory opt-in attributes).  Call once per device,
 * with that device current, outside stream capture.
 * Replaces actlize_la_ppu15_configure / actlize_la_ppu10_configure
 * (csrc/backends/ppu15/launch.cu:7-12, csrc/backends/ppu10/launch.h:5). */
int actlize_la_sm100_configure(void);

/* Static shape policy: kernel configuration id for a geometry; host metadata only, no
 * device access, no gate values.  Returns a negative value for an unsupported geometry.
 * Replaces actlize_la_ppu10_core_route_v2 (csrc/backends/ppu10/launch.h:9-10). */
int actlize_la_sm100_select(int batch, int sequence, int key_heads, int value_heads, int gate_fp32);

/* Bytes of caller-owned scratch that forward_prepared needs for this geometry and
 * configuration (the WY factors of every chunk); negative for an unsupported geometry.
 * Replaces the Python-side workspace table gdn_core_workspace_specs
 * (actlize_la/serving/gdn_core.py:14-22). */
long long actlize_la_sm100_workspace_bytes(int batch, int sequence, int key_heads, int value_heads,
                                           int config);

/* Complete forward on caller-owned buffers: prepare kernel (per-chunk gate prefix, decay-masked
 * K.K^T, unit-lower-triangular inverse, WY factors) followed by the sequential chunk walk.
 * `config` is the value returned by actlize_la_sm100_select: kernel family in bits 0..3, number of
 * sequence segments in bits 8..15, number of parallel sub-segments of the walk in bits 16..19 (tcgen05 family only;
 * 0 or 1 = off, at most 8).  With P parallel sub-segments P CTAs walk each (batch, value head) at the same time, every
 * one from a zero state and on into the leading chunks of the next piece that its state still reaches; this is exact
 * to exp(-40) of the state for heads whose pieces decay below exp(-40) within their own length and whose tokens
 * satisfy 0 <= beta |k|^2 <= 2 (checked on the device from the gates and the prepare kernel's K K^T diagonal, no
 * host read); any other head is walked by one CTA as without the split.  With more than one segment the prepare kernels and walks of the segments
 * behind the first run on two library-owned streams that are forked from and joined back into `stream` with
 * events (so the call stays asynchronous and capturable); those streams and events exist once per device,
 * therefore two segmented calls on the same device must not be in flight at the same time on different streams.
 * Replaces actlize_la_ppu15_forward_prepared / actlize_la_ppu10_forward_prepared
 * (csrc/backends/ppu15/launch.h:12-17, csrc/backends/ppu10/launch.h:11-14). */
int actlize_la_sm100_forward_prepared(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial, void* output, float* final_state,
    void* workspace, long long workspace_bytes,
    int batch, int sequence, int key_heads, int value_heads, int gate_fp32, int config,
    void* stream);

/* Host-buffer convenience used for end-to-end measurement and by callers without device
 * memory management: copies the host tensors to the device, runs forward_prepared and copies
 * output / final state back, all on `stream`, then synchronises that stream.
 * `device_arena` is caller-owned device memory of at least
 * actlize_la_sm100_host_arena_bytes(...) bytes.  The sequence is cut into segments (the configuration's count, or
 * four / two of the entry's own choice for the tcgen05 family when the configuration names one) whose transfers in
 * both directions overlap the computation of their neighbours on library-owned copy streams.  Follows the pack -> forward_prepared ->
 * scatter shape of the reference's prefill adapter (csrc/serving/prefill.cu:196-255). */
long long actlize_la_sm100_host_arena_bytes(int batch, int sequence, int key_heads, int value_heads,
                                            int gate_fp32, int has_initial, int has_final,
                                            int config);
int actlize_la_sm100_forward_host(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial, void* output, float* final_state,
    void* device_arena, long long device_arena_bytes,
    int batch, int sequence, int key_heads, int value_heads, int gate_fp32, int config,
    void* stream);

/* Sequence-parallel helpers (no counterpart in the reference, which has no multi-device
 * path; the affine composition rule is that of csrc/gdn_chunk/gdn_scan_stage2.cu:4-8).
 * state_out[b,h] = transition[b,h] @ state_in[b,h] + offset[b,h] for [B*Hv] FP32 128x128
 * blocks: carries a segment's incoming state across its affine map. */
int actlize_la_sm100_apply_transition(const float* transition, const float* offset,
                                      const float* state_in, float* state_out,
                                      int blocks, void* stream);

/* The exclusive scan of a rank's incoming state in one launch: `pairs` is FP32 [n_pairs][2][blocks][128][128] with the
 * (transition, offset) of earlier rank j at [j] (the transition of pair 0 is not read: the first rank contributes
 * its true outgoing state as offset 0); incoming = fold over j of (transition_j @ incoming + offset_j).  When
 * `outgoing` is not NULL it receives my_transition @ incoming + my_offset.  A transition block of exact zeros (a
 * segment that forgets its incoming state) costs a scan of the block instead of a product. */
int actlize_la_sm100_fold_transitions(const float* pairs, int n_pairs, const float* my_transition,
                                      const float* my_offset, float* incoming, float* outgoing,
                                      int blocks, void* stream);

/* ---- the steps either side of the forward (memory-bound, one streaming kernel each) ---- */

/* Step before: from a fused projection row [q heads | k heads | v heads] x 128 BF16 per token
 * (row stride in elements), raw gate inputs a, b [tokens, Hv] BF16 and per-head A_log, dt_bias FP32:
 * q,k <- x * rsqrt(sum x^2 + 1e-6) per head vector, v copied, g = -exp(A_log) * softplus(a + dt_bias)
 * (FP32, natural log), beta = sigmoid(b) (BF16).  Outputs are the contiguous gdn_forward inputs.
 * Replaces the packing kernel of the reference's prefill adapter (csrc/serving/prefill.cu:45-70,
 * csrc/serving/runtime.cuh:48-52). */
int actlize_la_sm100_prepare_inputs(
    const void* mixed, long long mixed_row_stride, const void* a, const void* b, const float* a_log,
    const float* dt_bias, void* q, void* k, void* v, float* g, void* beta, long long tokens,
    int key_heads, int value_heads, void* stream);

/* Single-token decode step on the same FP32 [B,Hv,128,128] K-by-V state, updated in place:
 * S <- exp(g) S; d = beta (v - k^T S); S <- S + k d^T; out = q^T S / sqrt(128).
 * q,k [B,Hk,128], v,out [B,Hv,128] BF16, g,beta [B,Hv].  Equals gdn_forward with T = 1.
 * Replaces the recurrent kernel of the reference's serving library (csrc/serving/gdn.cu:152). */
int actlize_la_sm100_decode_step(
    const void* q, const void* k, const void* v, const void* g, const void* beta, float* state, void* output,
    int batch, int key_heads, int value_heads, int gate_fp32, void* stream);

/* Speculative-decoding pair on the same K-by-V state (the reference's verify / commit, csrc/serving/gdn.cu:152-217 and
 * 255-300, without its slot pool and transaction records): verify_step runs `width` (1..64) draft tokens per
 * request through the recurrence, q,k [B,W,Hk,128], v [B,W,Hv,128], g,beta [B,W,Hv], reads `state` without
 * writing it, and returns the outputs [B,W,Hv,128] BF16 and delta_t = beta_t (v_t - k_t^T S) as FP32 [B,W,Hv,128];
 * commit_step then applies the first counts[b] (int32 on the device, clamped to 0..width) recorded updates
 * S <- e^{g_t} S + k_t delta_t^T in place.  verify + commit of all W tokens equals W decode steps bit for bit. */
int actlize_la_sm100_verify_step(
    const void* q, const void* k, const void* v, const void* g, const void* beta, const float* state, void* output,
    float* delta, int batch, int width, int hk, int hv, int gate_fp32, void* stream);
int actlize_la_sm100_commit_step(const void* k, const void* g, const float* delta, const int* counts, float* state,
                                 int batch, int width, int hk, int hv, int gate_fp32, void* stream);

/* Step after: out = y * rsqrt(mean(y^2) + 1e-6) * weight * silu(z) per 128-wide row, BF16.
 * Replaces rmsnorm_gated (csrc/output_gate/output_gate.cu:4-5,73-92). */
int actlize_la_sm100_rmsnorm_gated(const void* y, const void* z, const void* weight, void* out,
                                   long long rows, void* stream);

/* Step after, second half: the output projection C[M,N] = A[M,K] W[N,K]^T with BF16 operands, FP32 accumulation and
 * a BF16 result; A row-major, W in the Linear layout [N][K], C row-major; K and N multiples of 8, all pointers
 * 16-byte aligned.  One tcgen05 kernel (128 x 128 tiles, TMA-fed, accumulator in tensor memory); call
 * actlize_la_sm100_configure once per device first.
 * Replaces out_proj_gemm / out_proj_gemm_cutlass (csrc/output_gate/output_gate.cu, output_gate_cutlass.cu;
 * docs/OUTPUT_GATE.md:17-24). */
int actlize_la_sm100_out_proj(const void* a, const void* w, void* c, int m, int n, int k, void* stream);

/* Diagnostic word written by a kernel whose bounded wait ran out (all waits on barriers are
 * bounded; a kernel that gives up drains, frees its tensor memory and returns; its output rows and
 * final state are then incomplete): status4[0] = 0 when healthy else a failure code, [1] block index,
 * [2] wait site, [3] chunk.  Synchronises the device; `reset` != 0 clears the word.  Counterpart of the
 * per-request `errors[]` status of the reference's serving ABI (csrc/serving/abi.h:8-17). */
int actlize_la_sm100_device_status(int* status4, int reset);

/* The same record WITHOUT synchronising: the failing kernel also writes it to a page of pinned host
 * memory that configure() maps into the device (cudaHostRegister of library-owned storage; nothing is
 * allocated), and this call only reads that page.  A caller polls it after its own synchronisation, or
 * before its next launch to learn about an earlier one; all zero when healthy or when configure() has not
 * run on the current device.  Cleared by actlize_la_sm100_device_status(..., 1).  The forward entries
 * stay fire-and-forget; checking this word is the caller's part of failing closed. */
int actlize_la_sm100_last_failure(int* status4);

/* Diagnostic counters of the parallel walk (config bits 16..19), summed over the launches since the last reset:
 * counts2[0] = (batch, value head) walks that were split over several CTAs, counts2[1] = walks that one CTA did alone
 * because a sub-segment does not decay below exp(-40) within its length or a token is not a contraction.
 * Synchronises the device; `reset` != 0 clears the counters.  No counterpart in the reference (its kernels never
 * split a head's walk over the sequence). */
int actlize_la_sm100_walk_plan_counts(int* counts2, int reset);

/* Failure-detection self-test: launches one small kernel whose bounded wait can never be satisfied
 * (an mbarrier nothing arrives on, a few thousand polls).  The kernel gives up, writes
 * (1, 0, 99, tag) to the status word read by actlize_la_sm100_device_status and ends normally: the
 * context stays usable.  No counterpart in the reference, whose kernels wait without a limit. */
int actlize_la_sm100_selftest_wait_timeout(int tag, void* stream);

/* Failure-detection self-test of the chunk walk itself: launches the tcgen05 walk over a workspace that an
 * earlier forward_prepared call (configuration 1, one segment, same inputs) has filled, with a TMA producer
 * that stops feeding it after the first chunk and with the poll limit of the bounded waits lowered for this
 * launch (the limit travels on `stream` in front of and behind the kernel; run nothing else on the device
 * meanwhile).  Every role of the real kernel runs out of its wait or sees the CTA-wide flag; the CTAs drain,
 * free their tensor memory and return; the status record holds code 1.  `output` receives unspecified rows:
 * pass a scratch buffer.  Needs at least two chunks (sequence > 64). */
int actlize_la_sm100_selftest_walk_stall(
    const void* q, const void* k, const void* v, const void* g, const void* beta, void* output,
    void* workspace, long long workspace_bytes, int batch, int sequence, int key_heads, int value_heads,
    int gate_fp32, void* stream);

/* The forward on the raw projection outputs of the layer: the step before the path (Q/K L2-normalisation, gate
 * activation g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b); csrc/serving/prefill.cu:45-70,
 * csrc/serving/runtime.cuh:48-52) is done inside the tcgen05 prepare kernel instead of by a kernel of its own
 * (actlize_la_sm100_prepare_inputs): `mixed` is BF16 [B*T][mixed_row_stride] with the row layout
 * [Hk q vectors | Hk k vectors | Hv v vectors] x 128, `a` and `b` are BF16 [B*T][Hv], `a_log`, `dt_bias` FP32 [Hv].
 * Same results, bit for bit, as prepare_inputs followed by forward_prepared with an FP32 gate.  `config` as returned
 * by actlize_la_sm100_select (tcgen05 configuration, segments allowed, no stage bits); the workspace
 * (actlize_la_sm100_projections_workspace_bytes) also holds the normalised queries and keys for the walk.  Rows behind a batch
 * element's end inside its last chunk are the next element's tokens and meet exact zeros: inputs must be finite. */
long long actlize_la_sm100_projections_workspace_bytes(int b, int t, int hk, int hv, int config);
int actlize_la_sm100_forward_projections(
    const void* mixed, long long mixed_row_stride, const void* a, const void* b_act, const float* a_log,
    const float* dt_bias, const float* initial, void* output, float* final_state,
    void* workspace, long long workspace_bytes,
    int b, int t, int hk, int hv, int config, void* stream);

/* Packed variable-length sequences: q,k [1,total,Hk,128], v [1,total,Hv,128], g/beta [1,total,Hv] hold n_seqs
 * sequences back to back; cu_seqlens_host[0..n_seqs] (HOST integers, 0 = first, total = last, non-decreasing)
 * marks the boundaries; initial_states / final_states are FP32 [n_seqs,Hv,128,128] (nullable).  Every sequence
 * is chunked from its own start, an empty sequence passes its state through.  The reference has no such entry:
 * its serving prefill pads the requests into a fixed [R,W] batch first (csrc/serving/prefill.cu:196-255,
 * csrc/serving/abi.h:48-56); this entry removes the padding.  Two launches (tcgen05 prepare + walk) on `stream`
 * plus one small host-to-device copy of the offsets table (from pageable memory: not for stream capture).
 * Rows behind a sequence's end inside its last chunk are the next sequence's tokens; they are multiplied by
 * exact zeros, so all inputs must be finite.  `workspace` needs actlize_la_sm100_varlen_workspace_bytes(...)
 * bytes, 256-byte aligned.  Returns 0 or a cudaError_t value. */
long long actlize_la_sm100_varlen_workspace_bytes(long long total_tokens, int n_seqs, int hk, int hv);
int actlize_la_sm100_forward_varlen(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial_states, void* output, float* final_states,
    void* workspace, long long workspace_bytes,
    const int* cu_seqlens_host, int n_seqs, int hk, int hv, int gate_fp32, void* stream);

/* The packed forward with the offsets on the DEVICE: cu_seqlens_device[0..n_seqs] are int32 in device memory, as a
 * serving scheduler produces them; nothing is read on the host, nothing is allocated, and the call consists of kernel
 * launches only (a one-thread kernel builds the offsets table, then the two tcgen05 kernels), so it can be captured
 * in a CUDA graph.  `total_tokens` is the token dimension of the tensors.  Offsets are forced into
 * 0 <= ... <= total_tokens and made non-decreasing on the device; tokens behind the last offset are not written.
 * Grids and workspace are sized for the upper bound ceil(total/64) + n_seqs chunks
 * (actlize_la_sm100_varlen_workspace_bytes already returns that). */
int actlize_la_sm100_forward_varlen_device(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial_states, void* output, float* final_states,
    void* workspace, long long workspace_bytes,
    const int* cu_seqlens_device, int n_seqs, long long total_tokens, int hk, int hv, int gate_fp32, void* stream);

/* The same forward for callers that cannot allocate device memory (no counterpart in the
 * reference): the workspace is a fixed array inside the library instead of a caller buffer.
 * Meant for plugins inside a host framework that owns all allocations, or loops where a
 * cudaMalloc is not acceptable.  B*Hv*ceil(T/64) must not exceed
 * ACTLIZE_LA_SM100_STATIC_SCRATCH_MAX_BLOCKS, otherwise the call returns
 * ACTLIZE_LA_SM100_ERROR_SCRATCH_TOO_SMALL and launches nothing.  The first call on a device does a
 * one-time set-up there: make it before any stream capture.  All calls share the array, so calls
 * that overlap on the GPU race; issue them one after the other.  Allocates nothing. */
#define ACTLIZE_LA_SM100_STATIC_SCRATCH_MAX_BLOCKS 64
#define ACTLIZE_LA_SM100_ERROR_SCRATCH_TOO_SMALL (-2)
int actlize_la_sm100_forward_static_scratch(
    const void* q, const void* k, const void* v, const void* g, const void* beta,
    const float* initial, void* output, float* final_state,
    int batch, int sequence, int key_heads, int value_heads, int gate_fp32, int config,
    void* stream);

/* Number of kernel launches one forward_prepared call issues for this configuration. */
int actlize_la_sm100_launches_per_forward(int config);

#ifdef __cplusplus
}
#endif
#endif /* ACTLIZE_LA_SM100_H_ */
