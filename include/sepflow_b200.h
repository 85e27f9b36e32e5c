/*
 * sepflow_b200 -- C ABI of the B200 (sm_100a) cost-volume separation library.
 *
 * Drop-in boundary for the native ops of the reference's memory-saving separation path: each entry
 * point below does what one function of the reference's pybind11 module `MemorySaver` does
 * (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112), but takes plain device pointers and sizes
 * and writes into caller-provided output buffers.
 *
 * Conventions shared by all entry points
 *   - All tensors are contiguous row-major fp32 (argmax tensors int32) in device memory, 16-byte aligned.
 *       F1  (B, H1, W1, C)  image-1 features, already multiplied by 1/sqrt(C) by the caller (core/corr.py:419)
 *       F2  (B, H2, W2, C)  image-2 features of one pyramid level (core/corr.py:422)
 *     With S[b,i,j,u,v] = sum_c F1[b,i,j,c] * F2[b,u,v,c] (never stored):
 *       MA_u (B,H1,W1,2,H2)  [..,0,u] = max_v S   [..,1,u] = mean_v S
 *       MA_v (B,H1,W1,2,W2)  [..,0,v] = max_u S   [..,1,v] = mean_u S
 *       AM_u (B,H1,W1,1,H2), AM_v (B,H1,W1,1,W2)  int32 argmax, lowest index on ties
 *       A_u  (B,H1,W1,Kc,W2), A_v (B,H1,W1,Kc,H2) attention weights
 *       C_u  (B,H1,W1,Kc,H2) = sum_v S*A_u,  C_v (B,H1,W1,Kc,W2) = sum_u S*A_v
 *   - Outputs need no initialisation by the caller (the reference pre-fills with -inf / 0,
 *     MemorySaver_kernel_forward.cu:916-927; here every element is written by the kernels).
 *   - Limits: C a multiple of 4 with 4 <= C <= 256; any H1, W1, H2, W2, Kc >= 1 (Kc >= 0 is not
 *     needed by the max/avg entry points and ignored there).
 *   - `workspace` is scratch device memory of at least sfb_workspace_bytes(op, shape) bytes, 256-byte
 *     aligned; its first word is a device status word (0 = ok) that bounded device-side waits set
 *     instead of hanging.  Calls that share a workspace must be ordered on one stream.
 *   - `stream` is a cudaStream_t (NULL = legacy default stream).  Work is enqueued, not synchronised.
 *   - Return value: SFB_OK or an error code; sfb_last_error() has the message of this thread's last error.
 *   - The contraction runs on the tensor cores with TF32 operands (round-to-nearest) and FP32
 *     accumulation; the reference kernels use FP32 FMAs.
 */
#ifndef SEPFLOW_B200_H_
#define SEPFLOW_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sfb_shape {
  int32_t B, H1, W1, H2, W2, C, Kc;
} sfb_shape;

enum {
  SFB_OK = 0,
  SFB_ERR_INVALID_ARGUMENT = 1,    /* null pointer, misaligned pointer, non-positive size */
  SFB_ERR_UNSUPPORTED_SHAPE = 2,   /* C outside the supported range */
  SFB_ERR_WORKSPACE_TOO_SMALL = 3,
  SFB_ERR_CUDA = 4,                /* a CUDA runtime / driver call failed */
  SFB_ERR_DEVICE_TIMEOUT = 5       /* sfb_device_status: a bounded device-side wait gave up */
};

enum {
  SFB_OP_MAX_AVG_FORWARD = 0,          /* also covers the argmax variant */
  SFB_OP_COMPRESSION_FORWARD = 1,
  SFB_OP_MAX_ARGMAX_AVG_BACKWARD = 2,
  SFB_OP_COMPRESSION_BACKWARD = 3,
  SFB_OP_CORR_VOLUME = 4,
  SFB_OP_SEPARATION_BACKWARD = 5,
  SFB_OP_MAX_AVG_FORWARD_CF = 6,
  SFB_OP_COMPRESSION_CF = 7,               /* compression forward and attention backward, channels-first */
  SFB_OP_SEPARATION_FEATURE_BACKWARD_CF = 8,
  SFB_OP_SEPARATION_LEVEL_FORWARD = 9,
  SFB_OP_SEPARATION_LEVEL_BACKWARD = 10
};

/* Scratch bytes an op needs for `shape` (0 if the shape is invalid). */
size_t sfb_workspace_bytes(int op, const sfb_shape* shape);

/* Replaces MemorySaver.max_avg_forward (MemorySaver_cuda.cpp:10-21 -> MemorySaver_kernel_forward.cu:901-949). */
int sfb_max_avg_forward(const float* F1, const float* F2, float* MA_u, float* MA_v, const sfb_shape* shape,
                        void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  The same computation as sfb_max_avg_forward for callers that cannot
 * allocate device memory at all: a component that runs under a memory pool some other part of the program owns, a
 * real-time or serving loop that must never enter the allocator, a host application that hands this library nothing
 * but input and output buffers.  Its scratch is a fixed array of sfb_static_scratch_bytes() bytes (32 MiB) that is
 * part of the library image: every GPU that loads the library holds it until the process exits.
 *   - Shapes whose scratch need (sfb_workspace_bytes(SFB_OP_MAX_AVG_FORWARD, shape)) exceeds that size are
 *     rejected with SFB_ERR_UNSUPPORTED_SHAPE; BASELINE-style 48x64 feature maps with C=256 fit.
 *   - Set-up: the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current) and caches it; the first call of a thread that has no CUDA context current binds the device's
 *     primary context (cudaFree(0)).  Make those first calls before any stream capture begins.  Apart from that
 *     set-up no call allocates or frees memory, and no call uses an allocating library routine.
 *   - All calls on a device share the one array, so two calls that overlap on the GPU (different streams,
 *     or different threads) race; order them on one stream.  Contents left by an earlier call are never
 *     read: the status word is cleared and everything else is rewritten before use.
 *   - sfb_static_device_status reads the device status word of the built-in scratch of the current device (the
 *     first word of the array), like sfb_device_status does for a caller-provided workspace: 0, or the code a
 *     bounded device-side wait left when it gave up, in which case the outputs of that call are incomplete. */
int sfb_max_avg_forward_static(const float* F1, const float* F2, float* MA_u, float* MA_v, const sfb_shape* shape,
                               void* stream);
size_t sfb_static_scratch_bytes(void);
int sfb_static_device_status(void* stream, int32_t* device_status);

/* Replaces MemorySaver.max_argmax_avg_forward (MemorySaver_cuda.cpp:23-34 -> MemorySaver_kernel_forward.cu:962-1016). */
int sfb_max_argmax_avg_forward(const float* F1, const float* F2, float* MA_u, float* MA_v, int32_t* AM_u,
                               int32_t* AM_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                               void* stream);

/* Replaces MemorySaver.max_argmax_avg_backward (MemorySaver_cuda.cpp:55-78 ->
 * MemorySaver_kernel_max_avg_argmax_backward.cu:1198-1221).  gF1 (B,H1,W1,C), gF2 (B,H2,W2,C). */
int sfb_max_argmax_avg_backward(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                                const float* gMA_u, const float* gMA_v, float* gF1, float* gF2,
                                const sfb_shape* shape, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces MemorySaver.compression_forward (MemorySaver_cuda.cpp:36-53 -> MemorySaver_kernel_forward.cu:1029-1074)
 * for any Kc >= 1 (the reference kernel is compiled for Kc = 2 only, MemorySaver_kernel_forward.cu:20,1061). */
int sfb_compression_forward(const float* F1, const float* F2, const float* A_u, const float* A_v, float* C_u,
                            float* C_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                            void* stream);

/* Replaces MemorySaver.compression_backward (MemorySaver_cuda.cpp:80-103 ->
 * MemorySaver_kernel_compression_backward.cu:651-666).  gA_u like A_u, gA_v like A_v. */
int sfb_compression_backward(const float* F1, const float* F2, const float* A_u, const float* A_v,
                             const float* gC_u, const float* gC_v, float* gF1, float* gF2, float* gA_u,
                             float* gA_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                             void* stream);

/* Both backward ops in one call: gA_u, gA_v as sfb_compression_backward, and gF1 / gF2 = the SUM of the two
 * ops' feature gradients, which is what autograd forms from MemorySaver.compression_backward and
 * MemorySaver.max_argmax_avg_backward (functions/MemorySaver.py:71-105,140-177) when both act on the same
 * F1, F2.  One pair of gradient GEMMs instead of two. */
int sfb_separation_backward(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                            const float* gMA_u, const float* gMA_v, const float* A_u, const float* A_v,
                            const float* gC_u, const float* gC_v, float* gF1, float* gF2, float* gA_u,
                            float* gA_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                            void* stream);

/* The two halves of sfb_separation_backward, for autograd: the attention gradients are needed as soon as the
 * compression node runs its backward, the feature gradients can wait until the max/avg node's upstream
 * gradients exist.  Same definitions as above (functions/MemorySaver.py:140-177 and :71-105). */
int sfb_compression_attention_backward(const float* F1, const float* F2, const float* gC_u, const float* gC_v,
                                       float* gA_u, float* gA_v, const sfb_shape* shape, void* workspace,
                                       size_t workspace_bytes, void* stream);
int sfb_separation_feature_backward(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                                    const float* gMA_u, const float* gMA_v, const float* A_u, const float* A_v,
                                    const float* gC_u, const float* gC_v, float* gF1, float* gF2,
                                    const sfb_shape* shape, void* workspace, size_t workspace_bytes, void* stream);

/* Channels-first variants for the call site.  core/corr.py:428-457 permutes every op output from
 * (B,H1,W1,K,D) to (B,K,D,H1,W1) for the Conv3d attention and permutes the attention weights back; these
 * entry points read and write the (B,K,D,H1,W1) tensors directly (displacement-major, pixel fastest), so the
 * call site needs no permute copies.  Same mathematics as the entry points above:
 *   SEP_v (B,2,H2,H1,W1) = MA_u permuted, SEP_u (B,2,W2,H1,W1) = MA_v permuted, AM_u (B,H2,H1,W1), AM_v (B,W2,H1,W1),
 *   A_u (B,Kc,W2,H1,W1), A_v (B,Kc,H2,H1,W1), C_u (B,Kc,H2,H1,W1), C_v (B,Kc,W2,H1,W1); gradients alike.
 * AM_u / AM_v may both be NULL (inference). */
int sfb_max_argmax_avg_forward_cf(const float* F1, const float* F2, float* SEP_v, float* SEP_u, int32_t* AM_u,
                                  int32_t* AM_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                                  void* stream);
int sfb_compression_forward_cf(const float* F1, const float* F2, const float* A_u, const float* A_v, float* C_u,
                               float* C_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                               void* stream);
int sfb_compression_attention_backward_cf(const float* F1, const float* F2, const float* gC_u, const float* gC_v,
                                          float* gA_u, float* gA_v, const sfb_shape* shape, void* workspace,
                                          size_t workspace_bytes, void* stream);
int sfb_separation_feature_backward_cf(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                                       const float* gSEP_v, const float* gSEP_u, const float* A_u, const float* A_v,
                                       const float* gC_u, const float* gC_v, float* gF1, float* gF2,
                                       const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                                       void* stream);

/* Attention weights of the call site (core/corr.py:437-442 with the modules of core/sepflow.py:59-60):
 *   A = softmax over the displacement axis of Conv3d(2 -> Kc, kernel 3, padding 1)(X)
 * X (B,2,D,H1,W1) with `x_batch_stride` elements between samples (so X may be the first two channels of a
 * (B,K,D,H1,W1) tensor), weight (Kc,2,3,3,3), bias (Kc), A (B,Kc,D,H1,W1).  FP32 arithmetic.  1 <= Kc <= 64. */
int sfb_attention_forward(const float* X, int64_t x_batch_stride, const float* weight, const float* bias, float* A,
                          int32_t B, int32_t Kc, int32_t D, int32_t H1, int32_t W1, void* stream);
/* Its backward.  gA (B,Kc,D,H1,W1) holds dLoss/dA on entry and is overwritten with the logit gradients;
 * gX (B,2,D,H1,W1) = add + dLoss/dX, where `add` (shape of X, `add_batch_stride` elements between samples) may
 * be NULL; gweight (Kc,2,3,3,3), gbias (Kc).  Sums run in a fixed order (bit-reproducible).  `workspace` holds
 * per-block partial sums, sfb_attention_backward_workspace_bytes() bytes. */
size_t sfb_attention_backward_workspace_bytes(int32_t B, int32_t Kc, int32_t D, int32_t H1, int32_t W1);
int sfb_attention_backward(const float* X, int64_t x_batch_stride, const float* weight, const float* A, float* gA,
                           const float* add, int64_t add_batch_stride, float* gX, float* gweight, float* gbias,
                           int32_t B, int32_t Kc, int32_t D, int32_t H1, int32_t W1, void* workspace,
                           size_t workspace_bytes, void* stream);

/* One pyramid level of the call site in one call (core/corr.py:419-457, everything between the feature
 * permutes and the upsampling): max/avg sweep, attention weights, compression sweep, written straight into
 * the concatenated tensors
 *   SEP_u (B, 2+Kc, W2, H1, W1): channels 0,1 = max_u S, mean_u S;  2.. = C_v
 *   SEP_v (B, 2+Kc, H2, H1, W1): channels 0,1 = max_v S, mean_v S;  2.. = C_u
 * attention1 = (weight_u, bias_u) acts on SEP_u[:, :2] and gives A_u (B,Kc,W2,H1,W1); attention2 = (weight_v,
 * bias_v) on SEP_v[:, :2] gives A_v (B,Kc,H2,H1,W1).  A_u, A_v and (if not NULL) AM_u (B,H2,H1,W1), AM_v
 * (B,W2,H1,W1) are outputs the backward needs. */
int sfb_separation_level_forward(const float* F1, const float* F2, const float* weight_u, const float* bias_u,
                                 const float* weight_v, const float* bias_v, float* SEP_u, float* SEP_v,
                                 int32_t* AM_u, int32_t* AM_v, float* A_u, float* A_v, const sfb_shape* shape,
                                 void* workspace, size_t workspace_bytes, void* stream);
/* Backward of the level: from gSEP_u, gSEP_v (shapes of SEP_u, SEP_v) to gF1, gF2 and the gradients of the four
 * attention parameters.  Three contractions: the attention gradients (one sweep), then gF1 and gF2 from the
 * summed dLoss/dS of the max/avg and compression parts (one GEMM pair). */
int sfb_separation_level_backward(const float* F1, const float* F2, const float* weight_u, const float* weight_v,
                                  const float* SEP_u, const float* SEP_v, const int32_t* AM_u, const int32_t* AM_v,
                                  const float* A_u, const float* A_v, const float* gSEP_u, const float* gSEP_v,
                                  float* gF1, float* gF2, float* gweight_u, float* gbias_u, float* gweight_v,
                                  float* gbias_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                                  void* stream);

/* The same two calls on the model's own feature maps fmap1 (B,C,H1,W1), fmap2 (B,C,H2,W2) (shape->H1.. as above):
 * the transposition to channels-last and the multiplication of fmap1 by scale1 = 1/sqrt(C) that core/corr.py:419-422
 * does with permute().contiguous() happen inside the rounding copy, and the gradients come back as
 * gfmap1 (B,C,H1,W1) (chain rule through scale1 included) and gfmap2 (B,C,H2,W2).
 * Placement: with sep_channels = 0 the volumes are tensors of their own, as above.  Otherwise SEP_u / SEP_v (and
 * gSEP_u / gSEP_v) are tensors with `sep_channels` channels -- the concatenated outputs of all pyramid levels,
 * core/corr.py:473-475 -- and this level occupies channels sep_channel0 .. sep_channel0+2+Kc-1 (possible for the
 * level whose displacement range is the output's, i.e. level 0). */
int sfb_separation_level_forward_fmaps(const float* fmap1, const float* fmap2, float scale1, const float* weight_u,
                                       const float* bias_u, const float* weight_v, const float* bias_v, float* SEP_u,
                                       float* SEP_v, int32_t sep_channels, int32_t sep_channel0, int32_t* AM_u,
                                       int32_t* AM_v, float* A_u, float* A_v, const sfb_shape* shape, void* workspace,
                                       size_t workspace_bytes, void* stream);
int sfb_separation_level_backward_fmaps(const float* fmap1, const float* fmap2, float scale1, const float* weight_u,
                                        const float* weight_v, const float* SEP_u, const float* SEP_v,
                                        int32_t sep_channels, int32_t sep_channel0, const int32_t* AM_u,
                                        const int32_t* AM_v, const float* A_u, const float* A_v, const float* gSEP_u,
                                        const float* gSEP_v, float* gfmap1, float* gfmap2, float* gweight_u,
                                        float* gbias_u, float* gweight_v, float* gbias_v, const sfb_shape* shape,
                                        void* workspace, size_t workspace_bytes, void* stream);

/* Placement of one pyramid level's volumes into the concatenated outputs of the call site (core/corr.py:459-475:
 * F.interpolate(..., [D0,H1,W1], mode='trilinear', align_corners=True), then torch.cat over levels).  H1, W1 do not
 * change, so this is linear interpolation along the displacement axis, with torch's arithmetic.
 *   in (B,K,Dl,H1,W1) -> K consecutive channels of a (B,Ktot,D0,H1,W1) tensor: `out` points at the first of them in
 *   sample 0, `out_batch_stride` = Ktot*D0*H1*W1 elements.  Dl <= D0 (Dl == D0 copies).
 * The backward is the adjoint: gin (B,K,Dl,H1,W1) from the same channel slice of the output gradient. */
int sfb_upsample_displacement(const float* in, float* out, int64_t out_batch_stride, int32_t B, int32_t K, int32_t Dl,
                              int32_t D0, int32_t H1, int32_t W1, void* stream);
int sfb_upsample_displacement_backward(const float* gout, int64_t gout_batch_stride, float* gin, int32_t B, int32_t K,
                                       int32_t Dl, int32_t D0, int32_t H1, int32_t W1, void* stream);

/* Lookup on an aggregated 3D cost volume: the reference's CorrBlock1D (core/corr.py:513-624) for ONE of its two
 * volumes.  corr (B,dim,D,H1,W1) is the volume as the model holds it (core/sepflow.py:184-187); the pyramid over
 * the displacement axis (core/corr.py:543-548; levels 1..levels-1, level l = (B,dim,D>>l,H1,W1), back to back,
 * sfb_lookup_pyramid_bytes() bytes) is built once per volume; every refinement iteration then samples
 * 2*radius+1 linearly interpolated values per level around coord/2^l (core/corr.py:576-594):
 *   out (B, levels*dim*(2*radius+1), H1, W1), channel (l*dim + ch)*(2*radius+1) + tap.
 * coord (B,H1,W1) is one component of the model's coordinate tensor, `coord_batch_stride` elements between samples
 * (for coords (B,2,H1,W1): component pointer, stride 2*H1*W1).  clamp_unit != 0 clamps every sampling position to
 * [-1, 1] first, which is what the reference does for its first volume (core/corr.py:586).
 * 1 <= levels <= 8.  FP32 arithmetic. */
size_t sfb_lookup_pyramid_bytes(int32_t B, int32_t dim, int32_t D, int32_t H1, int32_t W1, int32_t levels);
int sfb_lookup_build_pyramid(const float* corr, float* pyramid, int32_t B, int32_t dim, int32_t D, int32_t H1,
                             int32_t W1, int32_t levels, void* stream);
int sfb_lookup_forward(const float* corr, const float* pyramid, const float* coord, int64_t coord_batch_stride,
                       float* out, int32_t B, int32_t dim, int32_t D, int32_t H1, int32_t W1, int32_t levels,
                       int32_t radius, int32_t clamp_unit, void* stream);
/* Gradient of the volume for upstream gradient gout (shape of out): gcorr (B,dim,D,H1,W1) is overwritten; gpyramid
 * (size of the pyramid) is scratch.  No atomics: bit-reproducible.  (No gradient for coord: the model detaches it,
 * core/sepflow.py:192.) */
int sfb_lookup_backward(const float* gout, const float* coord, int64_t coord_batch_stride, float* gcorr,
                        float* gpyramid, int32_t B, int32_t dim, int32_t D, int32_t H1, int32_t W1, int32_t levels,
                        int32_t radius, int32_t clamp_unit, void* stream);

/* Lookup on the 4D correlation volume without storing it: the call the reference's memory-saving block leaves
 * unimplemented (core/corr.py:491-510 raises NotImplementedError, then sketches
 * alt_cuda_corr.forward(fmap1, fmap2_l, coords / 2^l, radius) per level; alt_cuda_corr is RAFT's extension and is not
 * part of the reference checkout).  The result equals the dense block's lookup (core/corr.py:192-247): for every
 * image-1 pixel and level l, a (2r+1)x(2r+1) window of the level-l volume around coords / 2^l, bilinear with zero
 * padding (F.grid_sample, align_corners=True, core/utils/utils.py:110-118).
 *   F1 (B,H1,W1,C) and F2_levels[l] (B,H2[l],W2[l],C): features with channels innermost, as that call takes them
 *   (core/corr.py:500-501); level l of image 2 is avg_pool2d of level l-1 (core/corr.py:377-382);
 *   coords (B,2,H1,W1): (x, y) position in image 2 per image-1 pixel (core/sepflow.py:201);
 *   out (B, levels*(2r+1)^2, H1, W1), channel l*(2r+1)^2 + a*(2r+1) + b sampled at (x + a - r, y + b - r) -- the
 *   dense block's order (core/corr.py:214-231); every value times `scale` (the reference's 1/sqrt(C),
 *   core/corr.py:286,510).
 * F2_levels, H2, W2 are HOST arrays of `levels` entries.  C % 4 == 0, C <= 512, radius <= 4, H2[l], W2[l] >= 2;
 * feature and feature-gradient pointers 16-byte aligned.
 * FP32 arithmetic on unrounded features. */
int sfb_lookup4d_forward(const float* F1, const float* const* F2_levels, const int32_t* H2, const int32_t* W2,
                         int32_t levels, const float* coords, float* out, int32_t B, int32_t H1, int32_t W1, int32_t C,
                         int32_t radius, float scale, void* stream);
/* Gradients of the features for upstream gradient gout (shape of out): gF1 (shape of F1) is overwritten;
 * gF2_levels[l] (shape of F2_levels[l]) is zeroed and then accumulated with floating-point reductions, so its low
 * bits vary from run to run.  No gradient for coords: the model detaches them (core/sepflow.py:193). */
int sfb_lookup4d_backward(const float* F1, const float* const* F2_levels, const int32_t* H2, const int32_t* W2,
                          int32_t levels, const float* coords, const float* gout, float* gF1,
                          float* const* gF2_levels, int32_t B, int32_t H1, int32_t W1, int32_t C, int32_t radius,
                          float scale, void* stream);

/* Operand type of every contraction (the correlation sweeps and the gradient GEMMs) of the five ops, their fused and
 * channels-first forms and the level calls; accumulation is FP32 in every case, tensors stay FP32 in memory.
 *   SFB_OPERANDS_FP16 (default): features and the generated gradient operand rounded to FP16 -- the 10 mantissa bits
 *     of TF32 at twice its tensor-core rate.  FP16 has five exponent bits, so every tensor that becomes an operand is
 *     first multiplied by a power of two that brings its largest magnitude next to 1 (found on the device, applied
 *     exactly, undone when results are stored); results match the TF32 path to its own tolerance for data whose
 *     largest magnitudes lie within about 1e-12 .. 1e12.  Feature dimensions that are not multiples of 8 run as TF32.
 *   SFB_OPERANDS_TF32: rounded to TF32 (round to nearest), no scaling.
 *   SFB_OPERANDS_BF16: rounded to BF16 (8 mantissa bits; needs C % 8 == 0): the operand type BASELINE's bf16
 *     configuration asks for; gradients are then accurate to about 3e-3 instead of 3e-4.
 * The reference computes in FP32 only.  The initial setting can be chosen with SFB_OPERANDS=tf32|bf16|fp16 in the
 * environment.  The setting is process-wide (a backward runs on another thread than the
 * forward); sfb_set_sweep_operands returns the previous value, or -1 for an unknown one.  sfb_max_avg_forward_static,
 * sfb_corr_volume and the lookups always compute with TF32 / FP32 as documented at their declarations. */
enum { SFB_OPERANDS_TF32 = 0, SFB_OPERANDS_BF16 = 1, SFB_OPERANDS_FP16 = 2 };
int sfb_set_sweep_operands(int operands);
int sfb_get_sweep_operands(void);

/* Test aid with no counterpart in the reference ops: writes the dense volume S (B,H1,W1,H2,W2) of a
 * SMALL problem through the same tensor-core pipeline (the reference builds it with torch.matmul,
 * core/corr.py:286-289). */
int sfb_corr_volume(const float* F1, const float* F2, float* S, const sfb_shape* shape, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Synchronises `stream`, reads the workspace's device status word into *device_status and returns
 * SFB_OK if it is 0, SFB_ERR_DEVICE_TIMEOUT otherwise. */
int sfb_device_status(const void* workspace, void* stream, int32_t* device_status);

/* Test hook, no counterpart in the reference.  Every device-side wait in the kernels is bounded: when it runs out
 * the kernel writes a code to the status word (101 producer, 102 MMA issuer, 103 epilogue, 104 generator), all
 * roles of the CTA leave their loops, tensor memory is freed and the kernel returns by itself.  This call lets a
 * test see that path without faulting or hanging anything: `wait_limit_ns` replaces the 2 s limit of one wait
 * (0 = back to the default) and `drop_last_load` != 0 makes the correlation sweeps launched from now on leave out
 * the last block their producer would load, so that exactly one wait has nothing to wait for.  Process-wide; call
 * it with (0, 0) to return to normal operation. */
int sfb_debug_wait_timeout(uint64_t wait_limit_ns, int drop_last_load);

/* Per-kernel timing, off by default; no counterpart in the reference ops (its scripts time whole calls
 * with torch.utils.benchmark, scripts/test_maxavg_cuda.py:237-265).  While enabled, every kernel launch
 * is bracketed by CUDA events on the stream it is launched on.  sfb_kernel_timing_enable(1) starts a
 * fresh measurement, (0) stops; sfb_kernel_timing_read waits for the recorded events and returns the
 * accumulated device time and launch count of kernel `kernel` (0 <= kernel < sfb_kernel_timing_count()). */
int sfb_kernel_timing_enable(int on);
int sfb_kernel_timing_count(void);
int sfb_kernel_timing_read(int kernel, const char** name, double* total_ms, int64_t* launches);

const char* sfb_status_string(int code);
const char* sfb_last_error(void);
int sfb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SEPFLOW_B200_H_ */
