/*
 * b200_ops.h -- C ABI of libb200ops.so: hand-written sm_100a CUDA kernels for the ONNX
 * library-node hot path of DaCeML (MatMul / Gemm / Conv, Softmax / LogSoftmax, the
 * LayerNormalization and Gelu node chains, and the Add/Sub/Mul/Div/Pow/Sqrt/Erf/Relu nodes).
 *
 * Conventions (all entry points):
 *   - every tensor pointer is a DEVICE pointer to contiguous row-major fp32 unless a stride
 *     argument says otherwise; the caller owns every buffer, the library never allocates,
 *     frees or caches device memory, and never writes its inputs (one documented exception:
 *     b200_conv2d_static_f32 keeps its scratch in a fixed array inside the library and caches that
 *     array's address per device);
 *   - `stream` is a cudaStream_t passed as void*; all work is stream-ordered on it, the
 *     library never synchronises the host and never uses the default stream implicitly;
 *   - the return value is 0 on success or a negative B200_E* code; the message is available
 *     from b200_last_error_string() (thread-local). Nothing exits or throws across the ABI;
 *   - shapes/strides are int64_t counts of ELEMENTS.
 *
 * Each entry point replaces the GPU expansion of one DaCeML node type; the citation names the
 * `pure` expansion (path inside spcl/dace-onnx) whose results it must reproduce.
 */
#ifndef B200_OPS_H
#define B200_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

#define B200_OK 0
#define B200_EINVAL (-1)      /* bad pointer / shape / attribute */
#define B200_EUNSUPPORTED (-2) /* valid ONNX, but outside what this library implements */
#define B200_ECUDA (-3)       /* a CUDA runtime/driver call failed (launch, tensor-map encode) */
#define B200_EWORKSPACE (-4)  /* caller-provided workspace too small */
#define B200_EDEVICE (-5)     /* a kernel reported a bounded-wait expiry (see b200_device_status) */

/* Arithmetic mode of the contraction kernels. */
#define B200_MATH_FP32X3 0 /* tensor cores, 3xTF32 split (hi*hi + hi*lo + lo*hi), fp32 accumulate: fp32-accurate */
#define B200_MATH_TF32 1   /* tensor cores, single TF32 pass; ~1e-3 relative error, opt-in */
#define B200_MATH_FP32 2   /* CUDA-core fp32 FMA kernel; any shape/alignment */
#define B200_MATH_BF16 3   /* tensor cores, operands rounded to bf16 (8-bit mantissa), fp32 accumulate; ~4e-3 relative
                              error per product, opt-in. Dense (unbatched) MatMul / Gemm only, through b200_gemm_ws_f32
                              (both operands are converted into the workspace); batched contractions, the fused
                              attention and the convolution compute a B200_MATH_BF16 request in TF32, which is more
                              accurate. */

/* Fused epilogues of the contraction kernels: Y = epi(acc). */
#define B200_EPI_NONE 0          /* Y = acc */
#define B200_EPI_BIAS 1          /* Y = acc + bias[n]                      (MatMul -> Add, Gemm C, Conv B) */
#define B200_EPI_BIAS_RELU 2     /* Y = max(acc + bias[n], 0)              (-> Relu) */
#define B200_EPI_BIAS_GELU 3     /* t = acc + bias[n]; Y = t*0.5*(1+erf(t/sqrt(2)))  (Div,Erf,Add,Mul,Mul chain) */
#define B200_EPI_BIAS_RESIDUAL 4 /* Y = acc + bias[n] + residual[m,n]      (-> Add, Add) */
#define B200_EPI_SCALE 5         /* Y = acc * scale                        (-> Mul by a scalar constant) */

/* Elementwise binary / unary operator codes. */
#define B200_ADD 0
#define B200_SUB 1
#define B200_MUL 2
#define B200_DIV 3
#define B200_POW 4
#define B200_SQRT 0
#define B200_ERF 1
#define B200_RELU 2
#define B200_GELU 3 /* fused Div(sqrt2) -> Erf -> Add 1 -> Mul x -> Mul 0.5 chain */

B200_API int b200_version(void);
B200_API const char *b200_last_error_string(void);

/* Reads and clears the device-side status word that kernels with bounded waits set when a wait
 * expires (0 = clean). Synchronises the device: for tests and post-run checks, not hot paths. */
B200_API int b200_device_status(void);

/* Diagnostic: launches one tiny kernel (one warp) that waits on a barrier nothing will ever signal, with the
 * bounded wait all tensor-core kernels of this library use, limited to `budget_cycles` (1 .. 1e8) GPU clock cycles.
 * The wait expires, the kernel returns normally, and the next b200_device_status() reports B200_EDEVICE once
 * (role mask 0x8000) and is clean afterwards. Lets a deployment check the failure-reporting path without making
 * any real kernel fail. No counterpart in the reference (its library calls print and continue,
 * daceml/onnx/environments/cudnn.py / include/daceml_cudnn.h:15-22). */
B200_API int b200_selftest_wait_expiry(void *stream, int64_t budget_cycles);

/* ------------------------------------------------------------------------------------------
 * Contractions.
 * b200_gemm_f32 replaces ONNXMatMul (daceml/onnx/op_implementations/pure_implementations.py:130-235,
 * numpy matmul with batch broadcasting lowered to an einsum) and ONNXGemm (same file :433-459,
 * Y = A @ B^T + C with alpha=beta=1, transA=0, transB=1).
 *
 *   for every batch (bo, bi) in [0,batch_outer) x [0,batch_inner):
 *     Y_b[M,N] = epi( A_b[M,K] @ op(B_b) )
 *   A_b = A + bo*a_stride_outer + bi*a_stride_inner, rows lda apart (K contiguous);
 *   B_b likewise; trans_b=1: B_b is [N,K] with rows ldb apart; trans_b=0: B_b is [K,N];
 *   Y_b rows ldy apart. A batch stride of 0 broadcasts that operand (numpy semantics).
 *   bias has N entries (may be NULL for EPI_NONE/EPI_SCALE); residual addresses like Y.
 * The two-level batch lets attention heads be addressed in place ([B,S,heads,64] views).
 * ------------------------------------------------------------------------------------------ */
typedef struct b200_gemm_desc {
  int64_t batch_outer, batch_inner;
  int64_t M, N, K;
  int64_t lda, ldb, ldy;
  int64_t a_stride_outer, a_stride_inner;
  int64_t b_stride_outer, b_stride_inner;
  int64_t y_stride_outer, y_stride_inner;
  int32_t trans_b;
  int32_t epilogue;
  float scale;
  int32_t math_mode;
} b200_gemm_desc;

B200_API int b200_gemm_f32(void *stream, const b200_gemm_desc *desc, const float *A, const float *B,
                  const float *bias, const float *residual, float *Y);

/* The same contraction with device scratch, the way the reference's library-call expansions get a workspace
 * from their SDFG init hook (cudnn_implementations.py:281-301). With b200_gemm_workspace_bytes(desc) bytes of
 * 16-byte aligned scratch (0 = this call has no use for one: other modes, batched operands, or a product of
 * less than ~9 GFLOP, where the split's extra launch costs more than it saves), the fp32-accurate mode
 * (B200_MATH_FP32X3) splits
 * B once into its two TF32 halves there and runs a faster two-CTA kernel; results follow the same 3xTF32
 * arithmetic as b200_gemm_f32. A null or too small workspace is not an error in that mode: the call then behaves
 * exactly like b200_gemm_f32. B200_MATH_BF16 needs the workspace (it holds the bf16 copies of A and B) and returns
 * B200_EWORKSPACE without it. The scratch is only used during the call (stream-ordered). */
B200_API size_t b200_gemm_workspace_bytes(const b200_gemm_desc *desc);
B200_API int b200_gemm_ws_f32(void *stream, const b200_gemm_desc *desc, const float *A, const float *B,
                              const float *bias, const float *residual, float *Y, void *workspace,
                              size_t workspace_bytes);

/* Fused attention: out = Softmax(Q K^T * scale, axis=-1) V per (batch, head), the node pattern
 * MatMul -> Mul(constant) -> Softmax -> MatMul of the exported BERT graph (each node as in
 * pure_implementations.py:130-235, :87-89, :346-366) without writing the [seq, seq] scores to memory.
 * Q, K, V, out are [batch, seq, heads, head_dim] views given by element strides per row (token),
 * head and batch, head_dim contiguous -- e.g. slices of a fused QKV projection, and out laid out as
 * [batch, seq, hidden]. Implemented for math_mode TF32, head_dim 64, seq a multiple of 32 (any length),
 * scale > 0, 16-byte aligned Q/K/V with strides that are multiples of 4 and a 32-byte aligned out
 * with strides that are multiples of 8; b200_attention_supported() says whether a call qualifies,
 * anything else returns B200_EUNSUPPORTED and the caller runs the unfused nodes. */
typedef struct b200_attention_desc {
  int64_t batch, heads, seq, head_dim;
  int64_t q_row, q_head, q_batch;
  int64_t k_row, k_head, k_batch;
  int64_t v_row, v_head, v_batch;
  int64_t o_row, o_head, o_batch;
  float scale;
  int32_t math_mode;
} b200_attention_desc;

B200_API int b200_attention_supported(const b200_attention_desc *desc, const float *Q, const float *K,
                                      const float *V, const float *out);
B200_API int b200_attention_f32(void *stream, const b200_attention_desc *desc, const float *Q, const float *K,
                                const float *V, float *out);

/* ONNXConv (daceml/onnx/op_implementations/img_op_implementations.py:164-326): NCHW x OIHW
 * cross-correlation, group=1, dilation=1, symmetric zero padding (the padded form is what
 * daceml/transformation/pad_conv_fusion.py:77-95 folds into the node). bias may be NULL.
 * epilogue: B200_EPI_NONE / B200_EPI_BIAS / B200_EPI_BIAS_RELU.
 * workspace: b200_conv2d_workspace_bytes() bytes of device scratch (may be 0 -> NULL allowed). */
typedef struct b200_conv_desc {
  int64_t N, C, H, W;   /* input  X[N,C,H,W] */
  int64_t M, KH, KW;    /* filter W[M,C,KH,KW] */
  int64_t pad_h, pad_w; /* symmetric */
  int64_t stride_h, stride_w;
  int32_t epilogue;
  int32_t math_mode;
} b200_conv_desc;

B200_API size_t b200_conv2d_workspace_bytes(const b200_conv_desc *desc);
B200_API int b200_conv2d_f32(void *stream, const b200_conv_desc *desc, const float *X, const float *W,
                    const float *bias, float *Y, void *workspace, size_t workspace_bytes);

/* The same convolution with the constant work taken out of the call, the way the reference's cuDNN expansion sets
 * its filter / tensor descriptors up once in the SDFG init hook and only runs the convolution per call
 * (daceml/onnx/op_implementations/cudnn_implementations.py:281-301).
 *   b200_conv2d_prepare_filter_f32 repacks the OIHW filter W once (for B200_MATH_FP32X3 it also splits it into
 *     its two TF32 halves) into `filter`, b200_conv2d_filter_bytes(desc) bytes of 16-byte aligned device memory
 *     the caller keeps for as long as it runs this convolution; desc->N is ignored by both.
 *   b200_conv2d_prepared_f32 runs one convolution from a prepared filter. `flags` says in which layout the
 *     activations are: 0 = X and Y are NCHW as in ONNX; B200_CONV_X_NHWC = X is [N,H,W,C]; B200_CONV_Y_NHWC = Y is
 *     written as [N,OH,OW,M]. Between two convolutions of a stack the NHWC form saves the layout change the tensor
 *     cores need (only graph inputs / outputs pay it). NHWC is taken where b200_conv2d_nhwc_supported(desc) is 1
 *     (stride 1, C a multiple of 4 and >= 16, at most 64 output channels whose filter fits in shared memory, a
 *     tensor-core math mode); elsewhere a call with either flag returns B200_EUNSUPPORTED.
 *     `workspace`: b200_conv2d_prepared_workspace_bytes(desc, flags) bytes (0 with B200_CONV_X_NHWC).
 * Results are those of b200_conv2d_f32 (which is prepare + run on its own workspace). */
#define B200_CONV_X_NHWC 1
#define B200_CONV_Y_NHWC 2
B200_API size_t b200_conv2d_filter_bytes(const b200_conv_desc *desc);
B200_API int b200_conv2d_prepare_filter_f32(void *stream, const b200_conv_desc *desc, const float *W, void *filter,
                                            size_t filter_bytes);
B200_API int b200_conv2d_nhwc_supported(const b200_conv_desc *desc);
B200_API size_t b200_conv2d_prepared_workspace_bytes(const b200_conv_desc *desc, int flags);
B200_API int b200_conv2d_prepared_f32(void *stream, const b200_conv_desc *desc, int flags, const float *X,
                                      const void *filter, const float *bias, float *Y, void *workspace,
                                      size_t workspace_bytes);

/* Convolution for callers that cannot allocate device memory. No counterpart in the reference:
 * every GPU library call there gets its workspace from an SDFG init hook (cudaMalloc in
 * cudnn_implementations.py:281-297), which some embedders do not have -- generated code that owns
 * nothing but its argument pointers, or a service whose device memory is fixed at start-up.
 * Same arguments and results as b200_conv2d_f32 minus the workspace: the scratch is a fixed array of
 * B200_CONV_STATIC_SCRATCH_BYTES inside the library, resident on every GPU that loads the library
 * until the process exits. A convolution needing more scratch than that (see
 * b200_conv2d_workspace_bytes) is refused with B200_EWORKSPACE. The call itself allocates and frees
 * nothing. The first call on each device looks the array's address up (one cudaGetSymbolAddress,
 * cached per device); make that first call with the device current and before any stream capture
 * begins. All calls on a device share the array: calls that can overlap on the GPU (other streams or
 * threads) race; serialise them. Contents left by earlier calls never influence a result. */
#define B200_CONV_STATIC_SCRATCH_BYTES (32u << 20)
B200_API size_t b200_conv2d_static_scratch_bytes(void);
B200_API int b200_conv2d_static_f32(void *stream, const b200_conv_desc *desc, const float *X, const float *W,
                           const float *bias, float *Y);

/* ------------------------------------------------------------------------------------------
 * Row-wise kernels. A tensor is viewed as [outer, len, inner] around the reduced axis
 * (inner == 1 for the last axis).
 * ------------------------------------------------------------------------------------------ */
/* ONNXSoftmax, single numpy axis (pure_implementations.py:346-366): max, exp(x-max), sum, div. */
B200_API int b200_softmax_f32(void *stream, const float *x, float *y, int64_t outer, int64_t len, int64_t inner);
/* ONNXLogSoftmax (pure_implementations.py:594-616): (x-max) - log(sum(exp(x-max))). */
B200_API int b200_logsoftmax_f32(void *stream, const float *x, float *y, int64_t outer, int64_t len, int64_t inner);
/* ONNXReduceMean (pure_implementations.py:97-109): np.mean over one contiguous block of axes. */
B200_API int b200_reduce_mean_f32(void *stream, const float *x, float *y, int64_t outer, int64_t len, int64_t inner);
/* The 9-node LayerNormalization chain ReduceMean,Sub,Pow(2),ReduceMean,Add(eps),Sqrt,Div,Mul,Add
 * (the nodes of pure_implementations.py:97-109, :77-94, :59-74, :41-56 in that order) over the
 * last axis: y = (x-mean)/sqrt(mean((x-mean)^2)+eps)*gamma+beta. gamma/beta may be NULL. */
B200_API int b200_layernorm_f32(void *stream, const float *x, const float *gamma, const float *beta, float *y,
                       int64_t rows, int64_t len, float eps);

/* ------------------------------------------------------------------------------------------
 * Elementwise nodes with numpy broadcasting (pure_implementations.py:77-94 Add/Sub/Mul/Div,
 * :59-74 Pow). `shape` is the broadcast output shape (rank <= 8); a_strides/b_strides are element
 * strides of each operand in that shape, 0 on broadcast axes.
 * ------------------------------------------------------------------------------------------ */
B200_API int b200_binary_f32(void *stream, int op, const float *a, const float *b, float *c, int rank,
                    const int64_t *shape, const int64_t *a_strides, const int64_t *b_strides);
/* Sqrt (:41-56), Erf (:112-127), Relu (:462-474), and the fused Gelu chain. */
B200_API int b200_unary_f32(void *stream, int op, const float *x, float *y, int64_t numel);

/* Layout helper used either side of attention: out[b,h,s,d] = in[b,s,h,d] (ONNXTranspose
 * perm [0,2,1,3], pure_implementations.py:369-379). The same call undoes it with s,h swapped. */
B200_API int b200_transpose_0213_f32(void *stream, const float *x, float *y, int64_t d0, int64_t d1, int64_t d2,
                            int64_t d3);
/* out[c,r] = in[r,c] per batch (ONNXTranspose perm [1,0], the runtime Transpose(W) before MatMul). */
B200_API int b200_transpose_2d_f32(void *stream, const float *x, float *y, int64_t batch, int64_t rows, int64_t cols);

/* ONNXMaxPool as the reference's pure expansion accepts it (PureMaxPool2D,
 * daceml/onnx/op_implementations/img_op_implementations.py:29-140): 2-D, pads 0, ceil_mode 0, dilations 1, no Indices
 * output. x is [planes, H, W] (planes = N*C of an NCHW tensor), y is [planes, (H-kh)/sh+1, (W-kw)/sw+1]. Sits between
 * the convolutions of the reference's LeNet test (tests/pytorch/test_lenet.py:14-32). */
B200_API int b200_maxpool2d_f32(void *stream, const float *x, float *y, int64_t planes, int64_t H, int64_t W,
                                int64_t kh, int64_t kw, int64_t sh, int64_t sw);

#ifdef __cplusplus
}
#endif
#endif /* B200_OPS_H */
