/*
 * rwkvq.h -- C ABI of librwkvq.so: the quantized projection path of the RWKV-7
 * quantization toolkit AUXStar/rwkv7-quantization, written for NVIDIA B200 (sm_100a).
 *
 * Conventions (every entry point):
 *   - returns 0 (RWKVQ_OK) or a negative RWKVQ_E_* code; never throws, never allocates,
 *     never synchronizes the host with the device; rwkvq_last_error_string() describes the
 *     last failure on the calling thread;
 *   - pointers are DEVICE pointers unless the name says `host`; matrices are row-major with
 *     an explicit leading dimension in ELEMENTS (ld*); weights are [N, K] with K contiguous,
 *     exactly the layouts schemes.py / int4/quantize_int4.py / int8/quantize_int8.py of the
 *     reference write;
 *   - `stream` is a cudaStream_t passed as void* (0 = the legacy default stream); work is
 *     only enqueued;
 *   - `x_dtype` is RWKVQ_F16 or RWKVQ_BF16;
 *   - `div_mode` selects how the fp32 scale divisions (448/amax, amax/448, 127/amax, amax/127,
 *     x/awq) are evaluated: RWKVQ_DIV_FULL = PTX div.full.f32, which is what the reference's
 *     Triton kernels execute on a GPU; RWKVQ_DIV_IEEE = round-to-nearest, which is what the Triton CPU
 *     interpreter computes; RWKVQ_DIV_TORCH (rwkvq_actq_fp8 / rwkvq_actq_fp8_fused only) = the two-step forms torch
 *     evaluates on a GPU for `448.0 / amax` and `amax / 448.0` in prep_x_fp8 (fused_fp8_gemm.py:377, 389):
 *     rn(rn(1/amax) * 448) and rn(amax * rn(1/448)); checked bit for bit against the reference run on a B200.
 *
 * Each declaration names the reference function it replaces (file:line in the reference tree).
 */
#ifndef RWKVQ_H_
#define RWKVQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKVQ_OK 0
#define RWKVQ_E_BADARG (-1)    /* null pointer, unknown enum value                         */
#define RWKVQ_E_ALIGN (-2)     /* pointer or leading dimension not 16-byte aligned          */
#define RWKVQ_E_SHAPE (-3)     /* size outside what the entry point supports                */
#define RWKVQ_E_ARCH (-4)      /* device is not compute capability 10.x                     */
#define RWKVQ_E_LAUNCH (-5)    /* CUDA reported a launch / runtime error                    */
#define RWKVQ_E_TIMEOUT (-6)   /* a bounded device-side wait gave up                        */
#define RWKVQ_E_WORKSPACE (-7) /* caller-provided scratch is missing or too small           */

#define RWKVQ_F16 0
#define RWKVQ_BF16 1

#define RWKVQ_DIV_IEEE 0
#define RWKVQ_DIV_FULL 1
#define RWKVQ_DIV_TORCH 2 /* activation-quantization entry points only: see below */

/* flags of the W8A8 entry points */
#define RWKVQ_FLAG_AMAX_AFTER_BF16 1u /* amax over bf16-rounded x (reference M==1 kernel, fused_fp8_gemm.py:662) */
#define RWKVQ_FLAG_INT8_SHARED_WSCALE 2u /* k and v use r's weight scale (reference defect, fused_fp8_gemm.py:855-857) */
#define RWKVQ_FLAG_OUT_VIA_BF16 4u    /* round the result to bf16 before fp16 (fp8_ops.py:77-86)        */
#define RWKVQ_FLAG_WSCALE_PER_ROW 16u  /* w_scale holds N values, one per output row (schemes.py:26-34 "fp8_perchannel"; no reference kernel reads them) */
#define RWKVQ_FLAG_RELU2 32u       /* set by rwkvq_gemv_fp8_relu2 (ignored elsewhere): relu^2 in the epilogue, amax published  */
#define RWKVQ_FLAG_AMAX_GIVEN 64u  /* set by rwkvq_gemv_fp8_preamax (ignored elsewhere): quantize with the published amax      */
#define RWKVQ_FLAG_QUANT_FROM_BF16 8u /* quantize bf16(x) instead of x (the GEMM kernels read prep_x's bf16 copy, fused_fp8_gemm.py:248-250) */

int32_t rwkvq_version(void);
const char* rwkvq_last_error_string(void);
/* 0 when the current device can run this library (compute capability 10.x). */
int32_t rwkvq_device_ok(void);
/* number of this library's kernel launches enqueued by the calling process so far */
int64_t rwkvq_launch_count(void);

/* out[i] = a[i] / b[i] evaluated with div.full.f32 (div_mode FULL) or IEEE (test hook that lets a CPU
 * checker reproduce the hardware-defined division of the reference's Triton kernels). */
int32_t rwkvq_div_f32(const float* a, const float* b, float* out, int64_t n, int32_t div_mode, void* stream);

/* ---------------------------------------------------------------- activation preparation */

/* prep_x / prep_x_kernel (fused_fp8_gemm.py:30-79): out_bf16 = bf16(fp32(x) [/ awq]); amax[0] = max over the
 * whole call of |fp32(x) [/ awq]| (zeroed by this call first).  awq may be NULL.  out_bf16 may be NULL. */
int32_t rwkvq_prep_x(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, const float* awq,
                     void* out_bf16, int64_t ldo, float* amax, int32_t div_mode, void* stream);

/* prep3_x / prep3_x_kernel (fused_fp8_gemm.py:86-150): the same for xr, xk, xv in one launch; amax[0..2]. */
int32_t rwkvq_prep3_x(const void* xr, const void* xk, const void* xv, int32_t x_dtype, int64_t M, int64_t K,
                      int64_t ldx, const float* awq_r, const float* awq_k, void* out_r, void* out_k, void* out_v,
                      int64_t ldo, float* amax3, int32_t div_mode, void* stream);

/* prep_x_fp8 (fused_fp8_gemm.py:341-390): per-call amax, inv = 448 / max(amax, 1e-12) and scale[0] = amax / 448 as
 * torch evaluates them on a GPU (RWKVQ_DIV_TORCH), codes = e4m3_rn(clamp(x * inv, +-448)).  amax_scratch: one fp32
 * owned by the caller. */
int32_t rwkvq_prep_x_fp8(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes,
                         int64_t ldc, float* scale, float* amax_scratch, void* stream);

/* The activation half of linear_fp8_fused for M above the decode kernel's range (prep_x + the in-loop
 * quantization of fused_fp8_hwdot_gemm_kernel, fused_fp8_gemm.py:240-250) and of linear_fp8 (fp8_ops.py:71-75):
 * amax[0] = per-call amax (of bf16(x) with RWKVQ_FLAG_AMAX_AFTER_BF16), codes = e4m3_rn(clamp(v * inv, +-448)) with
 * inv = 448 / max(amax, 1e-12) under div_mode and v = bf16(x) with RWKVQ_FLAG_QUANT_FROM_BF16, else x;
 * scale (optional) = amax / 448 under div_mode. */
int32_t rwkvq_actq_fp8(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                       float* amax, float* scale, int32_t div_mode, uint32_t flags, void* stream);

/* rwkvq_actq_fp8 in ONE cooperative launch (no memset, no second kernel): same arguments and results.  `scratch`
 * (rwkvq_actq_fp8_fused_scratch_bytes() bytes, 4-byte aligned, ZEROED ONCE before its first use) carries the per-CTA
 * maxima, the rendezvous flags and an epoch word that every launch advances on the device: calls that are ordered on
 * a stream may share one scratch, and a call captured in a CUDA graph may be replayed any number of times (nothing
 * about the rendezvous is fixed on the host).  Calls that can overlap on the GPU need separate scratch buffers.
 * `status` (optional) receives RWKVQ_E_TIMEOUT if the bounded grid rendezvous gives up; zero the scratch again after
 * that.  rwkvq_actq_fp8_fused3 does the same for xr, xk, xv in one launch (the activation half of linear_rkv_fused,
 * fused_fp8_gemm.py:86-150 + 264-334): three code matrices, amax3[0..2]. */
int64_t rwkvq_actq_fp8_fused_scratch_bytes(void);
int32_t rwkvq_actq_fp8_fused(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes,
                             int64_t ldc, float* amax, float* scale, void* scratch, int64_t scratch_bytes,
                             int32_t* status, int32_t div_mode, uint32_t flags, void* stream);
int32_t rwkvq_actq_fp8_fused3(const void* xr, const void* xk, const void* xv, int32_t x_dtype, int64_t M, int64_t K,
                              int64_t ldx, uint8_t* codes_r, uint8_t* codes_k, uint8_t* codes_v, int64_t ldc,
                              float* amax3, void* scratch, int64_t scratch_bytes, int32_t* status, int32_t div_mode,
                              uint32_t flags, void* stream);

/* prep_x_int8 / _prep_x_int8_kernel (fused_fp8_gemm.py:687-731): per-ROW amax (floor 1e-12), s = 127/amax,
 * codes = trunc(clamp(x*s, -128, 127)), scales[m] = amax/127. */
int32_t rwkvq_prep_x_int8(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* codes,
                          int64_t ldc, float* scales, int32_t div_mode, void* stream);
/* prep3_x_int8 (fused_fp8_gemm.py:889-894: three prep_x_int8 calls) in ONE launch. */
int32_t rwkvq_prep3_x_int8(const void* xr, const void* xk, const void* xv, int32_t x_dtype, int64_t M, int64_t K,
                           int64_t ldx, int8_t* codes_r, int8_t* codes_k, int8_t* codes_v, int64_t ldc, float* scales_r,
                           float* scales_k, float* scales_v, int32_t div_mode, void* stream);

/* ---------------------------------------------------------------- W8A8 decode GEMV (M <= 32) */

/* linear_fp8_m1_fused / linear_fp8_fused (fused_fp8_gemm.py:600-679, 1020-1077, 219-257) for small M:
 * ONE launch that derives the per-call amax, quantizes x to e4m3 in the prologue and streams W once.
 * out[M,N] fp16 = fp16( (q(x) . W^T) * (amax/448 * w_scale[0]) ).  awq may be NULL. */
int32_t rwkvq_gemv_fp8(const void* x, int32_t x_dtype, const float* awq, const uint8_t* w, int64_t ldw,
                       const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                       int64_t ldx, int32_t div_mode, uint32_t flags, void* stream);

/* The FFN of a layer, decode: key projection -> relu_square -> value projection (rwkv7_fast_v3a.py:1109, 1136-1144).
 * rwkvq_gemv_fp8_relu2 is rwkvq_gemv_fp8 whose epilogue also applies the engine's relu_square to its fp16 result
 * (cuda/rwkv7_fast_ops_fp16.cu:787-799: h = fp16(max(y, 0)^2) in fp32 arithmetic), stores h and publishes max|h| (over
 * the bf16-rounded values with RWKVQ_FLAG_AMAX_AFTER_BF16, i.e. where the consumer takes its amax).
 * rwkvq_gemv_fp8_preamax is rwkvq_gemv_fp8 on x = h that quantizes with the published amax instead of deriving it: no
 * abs-max pass and no reduction in its prologue.  Results equal the three separate steps bit for bit.
 * ffn_scratch: 8 bytes of device memory owned by the caller, 8-byte aligned, ZEROED ONCE; the relu2 launch accumulates
 * into it, the preamax launch consumes and clears it, so one scratch serves every pair issued in order on a stream
 * (also under CUDA-graph replay).  Pass the same flags to both (RWKVQ_FLAG_AMAX_AFTER_BF16 for M == 1). */
int32_t rwkvq_gemv_fp8_relu2(const void* x, int32_t x_dtype, const uint8_t* w, int64_t ldw, const float* w_scale,
                             void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                             uint32_t flags, void* ffn_scratch, void* stream);
int32_t rwkvq_gemv_fp8_preamax(const void* x, int32_t x_dtype, const uint8_t* w, int64_t ldw, const float* w_scale,
                               void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                               uint32_t flags, void* ffn_scratch, void* stream);

/* The pair on INT8 weights, up to 8 rows.  INT8 activations carry one scale per ROW, so rwkvq_gemv_int8_relu2 publishes
 * max(h) per token row and rwkvq_gemv_int8_preamax quantizes every row of h with its own published maximum.
 * ffn_scratch: 64 bytes (the FP8 pair uses the first 8 of the same block), 8-byte aligned, zeroed once; left zero. */
int32_t rwkvq_gemv_int8_relu2(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale,
                              void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                              uint32_t flags, void* ffn_scratch, void* stream);
int32_t rwkvq_gemv_int8_preamax(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale,
                                void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                                uint32_t flags, void* ffn_scratch, void* stream);

/* The INT8 pair for many rows: rwkvq_tc_gemm_int8_relu2 is rwkvq_tc_gemm_int8 (tiled form, no accumulator output) with
 * relu_square in its epilogue; it folds the maximum of h per TOKEN ROW into row_max[M] (floats, zero before the call).
 * rwkvq_actq_int8_given then makes the codes and row scales of h with those maxima (elementwise, no abs-max pass) and
 * clears them, and rwkvq_tc_gemm_int8 finishes.  Same bits as projection -> relu_square -> projection. */
int32_t rwkvq_tc_gemm_int8_relu2(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                                 const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                 uint32_t flags, float* row_max, void* workspace, int64_t workspace_bytes, void* stream);
int32_t rwkvq_actq_int8_given(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* codes,
                              int64_t ldc, float* scales, float* row_max, int32_t div_mode, void* stream);

/* The same pair for many rows (prefill): rwkvq_tc_gemm_fp8_relu2 is rwkvq_tc_gemm_fp8 (tiled form, M >= 17) with
 * relu_square and the amax accumulation in its epilogue; rwkvq_actq_fp8_given then makes the codes of h with the
 * published amax -- purely elementwise, no abs-max pass and no grid rendezvous -- writes its own copies amax_out[0]
 * (and scale_out[0] = amax/448 under div_mode, optional) for the value GEMM and clears ffn_scratch. */
int32_t rwkvq_tc_gemm_fp8_relu2(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax,
                                const uint8_t* w, int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo,
                                int64_t M, int64_t N, int64_t K, int32_t div_mode, uint32_t flags, void* ffn_scratch,
                                void* workspace, int64_t workspace_bytes, void* stream);
int32_t rwkvq_actq_fp8_given(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes,
                             int64_t ldc, float* amax_out, float* scale_out, void* ffn_scratch, int32_t div_mode,
                             uint32_t flags, void* stream);

/* linear_rkv_fused / fused_rkv_fp8_kernel (fused_fp8_gemm.py:944-1017, 264-334): r, k, v in ONE launch;
 * three activations, three amax, three weight scales.  awq_r / awq_k may be NULL. */
int32_t rwkvq_gemv_fp8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const float* awq_r,
                           const float* awq_k, const uint8_t* wr, const uint8_t* wk, const uint8_t* wv, int64_t ldw,
                           const float* sr, const float* sk, const float* sv, void* out_r, void* out_k, void* out_v,
                           int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                           uint32_t flags, void* stream);

/* linear_int8_fused / fused_int8_gemm_kernel (fused_fp8_gemm.py:734-818) for small M: per-row activation
 * quantization in the prologue, exact int32 accumulation, out = fp16(float(acc) * (x_scale[m] * w_scale[0])).
 * acc_out (optional, int32 [M, ldacc]) receives the raw accumulators. */
int32_t rwkvq_gemv_int8(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale,
                        void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M, int64_t N, int64_t K,
                        int64_t ldx, int32_t div_mode, uint32_t flags, void* stream);

/* linear_rkv_int8_fused / fused_rkv_int8_kernel (fused_fp8_gemm.py:825-934). */
int32_t rwkvq_gemv_int8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const int8_t* wr,
                            const int8_t* wk, const int8_t* wv, int64_t ldw, const float* sr, const float* sk,
                            const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N,
                            int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags, void* stream);

/* Several decode projections with ONE call across the boundary (the per-layer loop of the engine, rwkv7_fast_v3a.py:819,
 * makes four such calls per layer and its host-side cost per call exceeds the kernels' run time at batch 1): the
 * descriptors are walked in order and each is launched exactly as rwkvq_gemv_fp8 / _fp8_rkv / _int8 / _int8_rkv would
 * launch it -- same kernels, same results.  Fields not used by a kind are ignored. */
#define RWKVQ_PROJ_FP8 0
#define RWKVQ_PROJ_FP8_RKV 1
#define RWKVQ_PROJ_INT8 2
#define RWKVQ_PROJ_INT8_RKV 3
typedef struct rwkvq_proj_desc {
    int32_t kind;            /* RWKVQ_PROJ_*                                   */
    int32_t x_dtype;         /* RWKVQ_F16 / RWKVQ_BF16                         */
    const void* x[3];        /* activations [M, ldx]; x[1], x[2] for r/k/v     */
    const float* awq[2];     /* FP8 r/k/v: optional per-channel divisors       */
    const void* w[3];        /* weights [N, ldw]                               */
    const float* w_scale[3];
    void* out[3];            /* fp16 [M, ldo]                                  */
    int64_t ldw, ldo, ldx, M, N, K;
    int32_t div_mode;
    uint32_t flags;
} rwkvq_proj_desc;
int32_t rwkvq_gemv_batch(const rwkvq_proj_desc* descs, int32_t count, void* stream);

/* ---------------------------------------------------------------- W8A8 GEMM on pre-quantized codes (any M) */

/* These run on mma.sync kernels and need no workspace: the weight-streaming decode kernel for M <= 32 (code tile in
 * shared memory), a register-streaming kernel for any other M; the tensor-memory entries further down compute the
 * same results on tcgen05 and are what the Python wrappers route larger M to.
 * The GEMM half of linear_fp8_fused / linear_fp8 (fused_fp8_gemm.py:219-257, fp8_ops.py:77-80):
 * out = fp16( (a_codes . W^T) * (a_scale * w_scale[0]) ), where a_scale = amax[0]/448 if amax_is_amax != 0
 * (div_mode applies) or a_scale = amax[0] taken as the scale itself otherwise. */
int32_t rwkvq_gemm_fp8(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax,
                       const uint8_t* w, int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M,
                       int64_t N, int64_t K, int32_t div_mode, uint32_t flags, void* stream);

/* The GEMM half of linear_rkv_fused / linear_rkv_int8_fused on codes (fused_rkv_fp8_kernel fused_fp8_gemm.py:264-334,
 * fused_rkv_int8_kernel :825-886): r, k, v in ONE launch of the weight-streaming decode kernel when M <= 32 and the
 * code tile fits shared memory (each CTA copies the M*K bytes of codes once: the activations are quantized once per
 * call, not once per CTA), three launches of the any-M kernel otherwise.  amax3 / scales_*: as amax / a_scales of the
 * single-matrix entries.  The single-matrix entries take the same decode route for such M.  Same results as three
 * single calls, bit for bit. */
int32_t rwkvq_gemm_decode_route(int64_t M, int64_t K); /* 1: M rows of K codes take the decode kernel */
int32_t rwkvq_gemm_fp8_rkv(const uint8_t* codes_r, const uint8_t* codes_k, const uint8_t* codes_v, int64_t lda,
                           const float* amax3, int32_t amax_is_amax, const uint8_t* wr, const uint8_t* wk,
                           const uint8_t* wv, int64_t ldw, const float* sr, const float* sk, const float* sv, void* out_r,
                           void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N, int64_t K, int32_t div_mode,
                           uint32_t flags, void* stream);
int32_t rwkvq_gemm_int8_rkv(const int8_t* codes_r, const int8_t* codes_k, const int8_t* codes_v, int64_t lda,
                            const float* scales_r, const float* scales_k, const float* scales_v, const int8_t* wr,
                            const int8_t* wk, const int8_t* wv, int64_t ldw, const float* sr, const float* sk,
                            const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N,
                            int64_t K, uint32_t flags, void* stream);

/* The GEMM half of linear_int8_fused (fused_fp8_gemm.py:734-782): codes int8 [M,K], a_scales fp32 [M]. */
int32_t rwkvq_gemm_int8(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                        const float* w_scale, void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M,
                        int64_t N, int64_t K, uint32_t flags, void* stream);

/* ---------------------------------------------------------------- tensor-memory kernels (tcgen05 + TMA)
 *
 * The same projections on the 5th-generation tensor cores.  `workspace` is caller-owned device scratch:
 * rwkvq_workspace_bytes() bytes (16-byte aligned), ZEROED ONCE before its first use; every launch leaves its
 * counters zero again, so one workspace serves any number of launches that are ordered on one stream.  Launches
 * that may overlap on the device (different streams) need separate workspaces.  The workspace also holds a status
 * word that a kernel sets to RWKVQ_E_TIMEOUT if one of its bounded waits gave up; rwkvq_workspace_status() reads
 * it (this one call synchronizes the device). */
int64_t rwkvq_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t nmat);
int32_t rwkvq_workspace_status(const void* workspace, int32_t* host_status);

/* linear_fp8_m1_fused / linear_fp8_fused (fused_fp8_gemm.py:600-679, 1020-1077) for M <= 16: one launch, activation
 * quantization by dedicated warps of the kernel, weights streamed by TMA into tcgen05.mma. */
int32_t rwkvq_tc_gemv_fp8(const void* x, int32_t x_dtype, const float* awq, const uint8_t* w, int64_t ldw,
                          const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                          int64_t ldx, int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes,
                          void* stream);
/* linear_rkv_fused (fused_fp8_gemm.py:944-1017) for M <= 16. */
int32_t rwkvq_tc_gemv_fp8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const float* awq_r,
                              const float* awq_k, const uint8_t* wr, const uint8_t* wk, const uint8_t* wv, int64_t ldw,
                              const float* sr, const float* sk, const float* sv, void* out_r, void* out_k, void* out_v,
                              int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                              uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream);
/* linear_int8_fused (fused_fp8_gemm.py:785-818) for M <= 16. */
int32_t rwkvq_tc_gemv_int8(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale,
                           void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M, int64_t N, int64_t K,
                           int64_t ldx, int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes,
                           void* stream);
/* linear_rkv_int8_fused (fused_fp8_gemm.py:897-934) for M <= 16. */
int32_t rwkvq_tc_gemv_int8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const int8_t* wr,
                               const int8_t* wk, const int8_t* wv, int64_t ldw, const float* sr, const float* sk,
                               const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M,
                               int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags, void* workspace,
                               int64_t workspace_bytes, void* stream);
/* GEMM on pre-quantized codes, any M (fused_fp8_hwdot_gemm_kernel fused_fp8_gemm.py:219-257, torch._scaled_mm
 * fp8_ops.py:77-80): at most 16 tokens (or at most 48 against K >= 8192 and few weight rows) stream the weights once
 * with a stream-K split (needs the workspace); everything else runs the tiled GEMM with tokens as the 128-row operand
 * (workspace optional, used for the status word only). */
int32_t rwkvq_tc_gemm_fp8(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax,
                          const uint8_t* w, int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M,
                          int64_t N, int64_t K, int32_t div_mode, uint32_t flags, void* workspace,
                          int64_t workspace_bytes, void* stream);
/* The GEMM half of linear_rkv_fused / fused_rkv_fp8_kernel (fused_fp8_gemm.py:264-334) on codes: r, k, v in ONE launch
 * (three code matrices [M, lda], amax3[0..2], three weights of one shape).  Same results as three rwkvq_tc_gemm_fp8. */
int32_t rwkvq_tc_gemm_fp8_rkv(const uint8_t* codes_r, const uint8_t* codes_k, const uint8_t* codes_v, int64_t lda,
                              const float* amax3, int32_t amax_is_amax, const uint8_t* wr, const uint8_t* wk,
                              const uint8_t* wv, int64_t ldw, const float* sr, const float* sk, const float* sv,
                              void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N, int64_t K,
                              int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream);
/* The GEMM half of linear_rkv_int8_fused / fused_rkv_int8_kernel (fused_fp8_gemm.py:825-886) on codes, one launch;
 * RWKVQ_FLAG_INT8_SHARED_WSCALE mirrors the reference (k and v scaled by r's weight scale). */
int32_t rwkvq_tc_gemm_int8_rkv(const int8_t* codes_r, const int8_t* codes_k, const int8_t* codes_v, int64_t lda,
                               const float* scales_r, const float* scales_k, const float* scales_v, const int8_t* wr,
                               const int8_t* wk, const int8_t* wv, int64_t ldw, const float* sr, const float* sk,
                               const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N,
                               int64_t K, uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream);
/* fused_int8_gemm_kernel (fused_fp8_gemm.py:734-782) on codes, any M. */
int32_t rwkvq_tc_gemm_int8(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                           const float* w_scale, void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc,
                           int64_t M, int64_t N, int64_t K, uint32_t flags, void* workspace, int64_t workspace_bytes,
                           void* stream);

/* ---------------------------------------------------------------- weight-only INT4 / INT8 GEMV (fp16 activations, M <= 16)
 *
 * Layouts are the ones int4/quantize_int4.py and int8/quantize_int8.py of the reference write: packed nibbles
 * [N, K/2] with the even k in the low nibble; fp32 scales / zeros [N, K/group]; MM4 / MM8 vectors mx, rx [K] and
 * my, ry [N].  x is fp16 [M, ldx]; results fp16 [M, ldo] with fp32 accumulation (what the reference's GEMV kernels
 * are written to compute, int4/fused_int4_gemm.py:27-171, int8/fused_int8_gemm.py:32-103). */

/* _int4_gemv_kernel / linear_int4_per_tensor (int4/fused_int4_gemm.py:27-69, int4/int4_ops.py:79-101):
 * signed nibble * scale[0]. */
int32_t rwkvq_gemv_int4_tensor(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const float* scale,
                               void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream);
/* _int4_affine_gemv_kernel / linear_int4_affine (int4/fused_int4_gemm.py:72-117, int4/int4_ops.py:104-130):
 * w = (u4 + 0.5) * ry[n] * rx[k] * 16 + my[n] + mx[k]. */
int32_t rwkvq_gemv_int4_affine(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const float* mx,
                               const float* rx, const float* my, const float* ry, void* out_f16, int64_t ldo, int64_t M,
                               int64_t N, int64_t K, void* stream);
/* _int4_groupwise_gemv_kernel / linear_int4_groupwise (int4/fused_int4_gemm.py:120-171, int4/int4_ops.py:133-157):
 * w = u4 * scale[n, k/group] + zero[n, k/group]; scales fp32 or fp16 (scale_is_f16), zeros fp32 or NULL
 * (symmetric: zero = -8 * scale).  Any group size that divides K; one warp per output row. */
int32_t rwkvq_gemv_int4_group_generic(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw,
                                      const void* scales, const float* zeros, int32_t scale_is_f16, int32_t group,
                                      void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream);
/* _int8_gemv_kernel / linear_int8_per_tensor (int8/fused_int8_gemm.py:32-61, int8/int8_ops.py:48-78). */
int32_t rwkvq_gemv_int8_w8a16(const void* x_f16, int64_t ldx, const int8_t* w, int64_t ldw, const float* scale,
                              void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream);
/* _int8_affine_gemv_kernel / linear_int8_affine (int8/fused_int8_gemm.py:64-103, int8/int8_ops.py:81-110):
 * w = (u8 + 0.5) * ry[n] * rx[k] * 256 + my[n] + mx[k]. */
int32_t rwkvq_gemv_int8_affine(const void* x_f16, int64_t ldx, const uint8_t* w_u8, int64_t ldw, const float* mx,
                               const float* rx, const float* my, const float* ry, void* out_f16, int64_t ldo, int64_t M,
                               int64_t N, int64_t K, void* stream);

/* The group-wise INT4 decode kernel (same reference lines as rwkvq_gemv_int4_group_generic): group 128 or 256, K a
 * multiple of 128, M <= 16, activations staged in shared memory (rwkvq_gemv_int4_group_smem_bytes() <= 200 KiB),
 * weights streamed once into mma.sync.m16n8k16.f16 fragments. */
int64_t rwkvq_gemv_int4_group_smem_bytes(int64_t M, int64_t K);
int32_t rwkvq_gemv_int4_group(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const void* scales,
                              const float* zeros, int32_t scale_is_f16, int32_t group, void* out_f16, int64_t ldo,
                              int64_t M, int64_t N, int64_t K, void* stream);
/* The same kernel with K cut into slices, for blocks of activations too large to sit beside a deep weight ring (many
 * rows and / or long rows: 16 rows of K = 16384 would otherwise take four passes over the weights).  Group 128, fp32
 * scales, K a multiple of 512, M <= 16.  Two launches: the streaming kernel over (row tiles) x (K slices) stores fp32
 * partial sums into `workspace`, a second kernel adds them in slice order (run-to-run identical).
 * rwkvq_gemv_int4_ksplit_slices(M, N, K): slices this form uses (1: the plain entry does the same in one launch;
 * 0: unsupported shape).  workspace: slices * M * N * 4 bytes, 16-byte aligned, contents irrelevant. */
int32_t rwkvq_gemv_int4_ksplit_slices(int64_t M, int64_t N, int64_t K);
int32_t rwkvq_gemv_int4_group_ksplit(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const float* scales,
                                     const float* zeros, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                     void* workspace, int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------- NVFP4 (W4A4, block-scaled)
 *
 * The reference has no NVFP4 code left; format and arithmetic follow its reports
 * (iterations/phase1_nvfp4_exploration/reports/03_fused_kernel_en.md:22-34, 07_quantization_toolchain_v2_en.md:18-25,
 * iterations/phase3_x5_residual_scheme/reports/11_fused_gemm_ops_en.md:20-26): e2m1 codes packed two per byte
 * (even k in the low nibble) [rows, K/2]; one e4m3 scale per 16 consecutive k [rows, K/16]; one fp32 tensor scale. */

/* Activation quantization: pts[0] = amax/2688; block scale = e4m3(clamp(max|x|_16 * 448/amax, 2^-6, 448));
 * code = e2m1_rn(x * (1/pts) / block scale).  amax_scratch: one fp32 owned by the caller. */
int32_t rwkvq_actq_nvfp4(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                         uint8_t* block_scales, int64_t lds, float* pts, float* amax_scratch, void* stream);
/* out = fp16((sum_k codeA*bsA * codeB*bsB) * a_pts[0] * w_tscale[0]) for M <= 16 rows, K a multiple of 128;
 * rwkvq_gemv_nvfp4_smem_bytes(M, K) must not exceed 200 KiB. */
int64_t rwkvq_gemv_nvfp4_smem_bytes(int64_t M, int64_t K);
int32_t rwkvq_gemv_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_block_scales, int64_t ldas,
                         const float* a_pts, const uint8_t* w_codes, int64_t ldw, const uint8_t* w_block_scales,
                         int64_t ldws, const float* w_tscale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                         void* stream);

/* The same quantization in ONE cooperative launch (amax, grid-wide rendezvous with a bounded wait, codes and scales;
 * scratch rules as for rwkvq_actq_fp8_fused: zeroed once, epoch advanced on the device, safe under graph replay).
 * block_scales (row-major) and block_scales_blocked (the order rwkvq_tc_gemm_nvfp4 takes, K a multiple of 64, buffer
 * of rwkvq_nvfp4_blocked_scale_bytes(M, K); rows past M are left unwritten) may each be NULL, not both.  scratch:
 * rwkvq_actq_nvfp4_fused_scratch_bytes() bytes owned by the caller, not shared by overlapping calls; status (may be
 * NULL) receives RWKVQ_E_TIMEOUT if the rendezvous gives up. */
int64_t rwkvq_actq_nvfp4_fused_scratch_bytes(void);
int32_t rwkvq_actq_nvfp4_fused(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes,
                               int64_t ldc, uint8_t* block_scales, int64_t lds, uint8_t* block_scales_blocked, float* pts,
                               void* scratch, int64_t scratch_bytes, int32_t* status, void* stream);

/* Decode projection in ONE launch, M <= 16, K a multiple of 512: the activation quantization above runs in the kernel's
 * prologue (same arithmetic: amax, tensor scale, block scales, codes) and the weights are streamed once; the result
 * equals rwkvq_actq_nvfp4 followed by rwkvq_gemv_nvfp4 up to the order of the fp32 additions.  Weight code rows and
 * weight scale rows 16-byte aligned.  rwkvq_gemv_nvfp4_fused_smem_bytes(M, K) must not exceed 224 KiB. */
int64_t rwkvq_gemv_nvfp4_fused_smem_bytes(int64_t M, int64_t K);
int32_t rwkvq_gemv_nvfp4_fused(const void* x, int32_t x_dtype, int64_t ldx, const uint8_t* w_codes, int64_t ldw,
                               const uint8_t* w_block_scales, int64_t ldws, const float* w_tscale, void* out_f16,
                               int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream);

/* Many-token NVFP4 projection on the block-scaled tensor cores (tcgen05 kind::mxf4nvf4, 16-wide blocks): the path
 * the reference's reports call "block-scaled NVFP4 MMAs" (11_fused_gemm_ops_en.md:20-26).  Same arithmetic and
 * operands as rwkvq_gemv_nvfp4 for any M, except that both scale arrays are given BLOCKED: 512-byte chunks
 * [ceil(rows/256)*2 row tiles of 128][K/64][(r%32)*16 + (r/32)*4 + (k/16)%4], the order in which the tensor core
 * takes them from tensor memory; rows past `rows` hold zero.  rwkvq_nvfp4_pack_scales converts row-major scales
 * [rows, K/16] (once per weight; per call for activations) into a buffer of rwkvq_nvfp4_blocked_scale_bytes(rows, K).
 * K must be a multiple of 256; code rows 16-byte aligned.  workspace (may be NULL) receives the status word read by
 * rwkvq_workspace_status: every wait in the kernel is bounded and a timeout is reported there. */
int64_t rwkvq_nvfp4_blocked_scale_bytes(int64_t rows, int64_t K);
int32_t rwkvq_nvfp4_pack_scales(const uint8_t* block_scales, int64_t lds, int64_t rows, int64_t K, uint8_t* blocked,
                                void* stream);
/* NVFP4 projection of one to four tokens in ONE launch: the cluster split-K kernel with the activation quantization
 * inside (each CTA quantizes its K slice, the abs-max crosses the cluster through distributed shared memory).  Same
 * bits as rwkvq_actq_nvfp4_fused followed by rwkvq_tc_gemm_nvfp4.  x: [M, ldx] fp16 / bf16, rows 16-byte aligned;
 * weights as for rwkvq_tc_gemm_nvfp4 (packed codes, BLOCKED scales).  Sizes for which ..._route() returns 1. */
int32_t rwkvq_tc_gemv_nvfp4_fused_route(int64_t M, int64_t N, int64_t K);
int32_t rwkvq_tc_gemv_nvfp4_fused(const void* x, int32_t x_dtype, int64_t ldx, const uint8_t* w_codes, int64_t ldw,
                                  const uint8_t* w_scales_blocked, const float* w_tscale, void* out_f16, int64_t ldo,
                                  int64_t M, int64_t N, int64_t K, void* stream);
/* 1 if rwkvq_tc_gemm_nvfp4 runs these sizes on the cluster split-K kernel (up to 256 tokens against few row tiles:
 * weights as the 128-row operand, K split across a thread-block cluster), 0 for the tiled form */
int32_t rwkvq_tc_gemm_nvfp4_cluster_route(int64_t M, int64_t N, int64_t K);
int32_t rwkvq_tc_gemm_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts,
                            const uint8_t* w_codes, int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale,
                            void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace,
                            int64_t workspace_bytes, void* stream);
/* rwkvq_tc_gemm_nvfp4 FUSED with the all-gather of a column-split projection (one kernel: tensor-core tiles and peer
 * stores).  Every result vector is also stored, by plain peer stores over NVLink, at the same offset behind
 * peer_out[p] -- this rank's column range in rank p's [M, ldo] buffer, aligned like out_f16 -- for p < npeers <= 7, so
 * the gather travels while the next tiles are computed.  When the whole grid has stored its tiles, `epoch` is
 * published (system-scope release) at peer_flag[p], this rank's slot in rank p's flag array; the receivers call
 * rwkvq_peer_wait.  The workspace is required (it counts finished CTAs); M, N > 0.  No TMA on peer memory. */
int32_t rwkvq_tc_gemm_nvfp4_push(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts,
                                 const uint8_t* w_codes, int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale,
                                 void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace,
                                 int64_t workspace_bytes, void* const* peer_out, void* const* peer_flag, int32_t npeers,
                                 uint32_t epoch, void* stream);

/* No counterpart in the reference.  FP8 projection of a few rows (up to 32) in ONE launch on the tensor-memory path,
 * for matrices with few 128-row tiles (N = 4096: attention output, FFN value): K is split across a thread-block
 * cluster, every CTA quantizes ITS K slice of the activations (the cluster exchanges the abs-max through distributed
 * shared memory), writes the e4m3 codes into the operand ring itself and the partial sums are added in rank order.
 * Same bits as rwkvq_actq_fp8_fused followed by rwkvq_tc_gemm_fp8, and measured slower than those two launches on
 * the 7.2B shapes (every cluster quantizes the whole block again), so the drop-in dispatcher does not take it; it
 * serves callers for whom one launch matters more than its duration.  rwkvq_tc_cluster_gemv_route(M, N, K) = 1 where
 * the form applies.  Flags: AMAX_AFTER_BF16, QUANT_FROM_BF16, WSCALE_PER_ROW, OUT_VIA_BF16. */
int32_t rwkvq_tc_cluster_gemv_route(int64_t M, int64_t N, int64_t K);
int32_t rwkvq_tc_cluster_gemv_fp8(const void* x, int32_t x_dtype, int64_t ldx, const uint8_t* w, int64_t ldw, const float* w_scale,
                                  void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int32_t div_mode, uint32_t flags,
                                  void* stream);

/* The same fusion for the FP8 W8A8 GEMM (rwkvq_tc_gemm_fp8 + all-gather in one kernel).  Only the tiled GEMM form can
 * carry it: rwkvq_tc_gemm_can_push(M, N, K) is 1 for the row counts it takes; the RELU2 flag is not accepted. */
int32_t rwkvq_tc_gemm_can_push(int64_t M, int64_t N, int64_t K);
int32_t rwkvq_tc_gemm_fp8_push(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                               int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                               int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes,
                               void* const* peer_out, void* const* peer_flag, int32_t npeers, uint32_t epoch, void* stream);
/* ... and for the INT8 W8A8 GEMM (rwkvq_tc_gemm_int8 without the accumulator output). */
int32_t rwkvq_tc_gemm_int8_push(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                                const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, uint32_t flags,
                                void* workspace, int64_t workspace_bytes, void* const* peer_out, void* const* peer_flag,
                                int32_t npeers, uint32_t epoch, void* stream);

/* No counterpart in the reference.  rwkvq_tc_gemm_fp8 for callers that cannot supply device scratch -- a host runtime
 * that owns every byte of device memory and forbids allocation inside its serving loop, or code running where
 * cudaMalloc is not allowed.  The scratch is an 8 MiB array built into the library on each GPU; no allocation happens
 * in this call or below it.  The first call on a device resolves the array's address and should be made outside
 * stream capture.  Only the stream-K form (few tokens against a matrix with too many 128-row tiles for the cluster
 * kernel) keeps partial sums there; such a call is refused (RWKVQ_E_WORKSPACE) when it needs more than 8 MiB; every
 * other shape is accepted.
 * The array is shared by all calls on a device, its header is re-cleared on `stream` by every call, and calls that
 * overlap on the GPU race on it.  rwkvq_tc_static_status copies its status word to the host (synchronizes). */
int32_t rwkvq_tc_gemm_fp8_static(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax,
                                 const uint8_t* w, int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo,
                                 int64_t M, int64_t N, int64_t K, int32_t div_mode, uint32_t flags, void* stream);
int32_t rwkvq_tc_static_status(int32_t* host_status);

/* ---------------------------------------------------------------- column-split projection across GPUs (NVLink peer memory)
 *
 * No counterpart in the reference (single process, single GPU).  The FFN key weight [F, C] is split by output rows
 * over `world` ranks (one process per GPU); every rank computes its [M, F/world] slice and the slices are gathered
 * along the features.  Every rank owns one buffer OUT [M, ld >= F] fp16 that its peers can address (exchange the
 * pointers once, e.g. through CUDA IPC handles) and one array of `world` 32-bit flags, zeroed once, also addressable
 * by the peers.  Per call, on one stream: (1) the projection entry point writes the rank's own columns straight into
 * OUT (out = OUT + rank * n_local, ldo = ld); (2) rwkvq_peer_signal stores `epoch` into flags[rank] of EVERY rank's
 * flag array (system-scope release behind a system-scope fence); (3) rwkvq_allgather_cols_pull waits, bounded, for
 * flags[s] == epoch of each source rank s and copies that rank's columns out of its OUT into the local OUT with
 * ordinary 16-byte peer loads.  `outs` and `flag_arrays` are HOST arrays of `world` device pointers in rank order.
 * Use a strictly increasing epoch per call and two OUT buffers in turn (a peer may still be reading the previous
 * call's columns while this rank computes the next).  A rank that never signals makes the pull give up after the
 * wait limit: RWKVQ_E_TIMEOUT in *status (device pointer; NULL = the per-device status word).  No TMA and no
 * multicast touches peer memory.
 * Set-up (the only entry points that allocate; not for the serving loop): rwkvq_peer_alloc returns `bytes` of zeroed
 * memory on the current device with its 64-byte CUDA IPC handle; rwkvq_peer_open maps another process's buffer from
 * such a handle -- call it with this process's own device current, the open sets up peer access between the two
 * devices; rwkvq_peer_close / rwkvq_peer_free undo them.  rwkvq_enable_peer_access(d) makes device d's ordinary
 * allocations of THIS process addressable from kernels of the current device (single-process use). */
int32_t rwkvq_peer_alloc(int64_t bytes, void** ptr_out, void* handle64_out);
int32_t rwkvq_peer_open(const void* handle64, void** ptr_out);
int32_t rwkvq_peer_close(void* ptr);
int32_t rwkvq_peer_free(void* ptr);
int32_t rwkvq_enable_peer_access(int32_t peer_device);
int32_t rwkvq_peer_signal(void* const* flag_arrays, int32_t rank, int32_t world, uint32_t epoch, void* stream);
int32_t rwkvq_allgather_cols_pull(void* const* outs, const uint32_t* my_flags, uint32_t epoch, int32_t rank, int32_t world,
                                  int64_t M, int64_t n_local, int64_t ld, int32_t* status, void* stream);
/* Receiver side of a pushed result (rwkvq_tc_gemm_nvfp4_push): waits on `stream`, bounded, until flags[r] == epoch for
 * every r != rank; a rank that never signals leaves RWKVQ_E_TIMEOUT in *status (NULL: the per-device status word). */
int32_t rwkvq_peer_wait(const uint32_t* my_flags, uint32_t epoch, int32_t rank, int32_t world, int32_t* status, void* stream);

/* ---------------------------------------------------------------- bounded waits, status, diagnostics
 *
 * No counterpart in the reference (its kernels have no device-side waits).  Every device-side wait of this library
 * (mbarriers of the tensor-memory kernels, staging copies of the decode GEMVs, the grid rendezvous of the one-launch
 * quantizers) gives up after a wall-time limit: 1.5 s by default, RWKVQ_WAIT_LIMIT_US in the environment (read once)
 * or rwkvq_set_wait_limit_us (0 restores the default) change it for launches made afterwards.  A kernel that gives up
 * records RWKVQ_E_TIMEOUT -- in the caller's status pointer / workspace where the entry point takes one, else in a
 * status word the library keeps on each device -- stops issuing work, waits (bounded) for its own copies in flight,
 * frees its tensor memory and returns; its results are then undefined.
 *   rwkvq_device_status   copies the per-device word to the host (synchronizes), optionally clearing it.
 *   rwkvq_selftest_timeout launches one CTA that waits, with limit_us, for an mbarrier phase nobody completes
 *                         (mode 0) or for a flag nobody writes (mode 1; scratch4 = 4 bytes of device memory) and must
 *                         leave RWKVQ_E_TIMEOUT in *status (device pointer) -- the give-up path without any fault. */
void rwkvq_set_wait_limit_us(int64_t microseconds);
int32_t rwkvq_device_status(int32_t* host_status, int32_t clear);
int32_t rwkvq_selftest_timeout(int32_t* status, void* scratch4, int64_t limit_us, int32_t mode, void* stream);
/* Profiling aids: a device buffer ([grid][8] uint64 for the decode GEMV, [grid][16] for the tensor-memory kernels) that
 * every later launch stamps with %globaltimer values at its CTAs' milestones; NULL (the default) switches them off.
 * The stamps are compiled into the kernels only when the library is built with -DRWKVQ_TRACE (build_ext.py --trace);
 * in a regular build these two calls have no effect. */
void rwkvq_gemv_set_trace(void* device_buffer);
void rwkvq_tc_set_trace(void* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* RWKVQ_H_ */
