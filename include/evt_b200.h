/* C-ABI of the B200 back end for EVT's fused operators.
 *
 * One "plan" = one fused node: a heavy op (GEMM, batched GEMM, softmax, LayerNorm, ... ,
 * CSR SpMM) plus its compiled epilogue.  The Python fuser creates the plan once, then
 * launches it with raw device pointers on a CUDA stream.  This boundary replaces, for the
 * reference, the CUTLASS-Python runtime calls made by its fused-op wrappers:
 *
 *   python/gtl/compiler/passes/evt_fuser.py:481-518, 605-642   plan.compile(...)      -> evtb_plan_create
 *   python/gtl/compiler/passes/evt_fuser.py:539-546, 674-680   operation.run(args, s) -> evtb_launch
 *   python/gtl/ops/reduce_apply_operation.py:44-86, 147-160    <op>_get_params + rt_module.run
 *                                                                                     -> evtb_launch
 *   python/gtl/ops/reduce_apply_operation.py:102-108           shared-memory opt-in   -> inside evtb_plan_create
 *   python/gtl/ops/spmm.py:40-43                               CSR as three pointers  -> operand order of SPMM plans
 *
 * Rules: every function returns an int status (0 = EVTB_OK); nothing throws; nothing
 * allocates device memory; nothing synchronises; launches only enqueue work on `stream`
 * and may be captured in a CUDA graph.  The caller owns all tensors, the workspace and the
 * status word.  Reduction targets must be pre-filled by the caller with the value
 * the code generator reports for the slot: 0 for sums, -inf for maxima (the reference zero-fills
 * them, evt_fuser.py:217-225).
 */
#ifndef EVT_B200_H_
#define EVT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct evtb_plan evtb_plan;
typedef void* evtb_stream; /* cudaStream_t */

enum evtb_status {
  EVTB_OK = 0,
  EVTB_EINVAL = 1,        /* bad descriptor: sizes, alignment, unknown kind */
  EVTB_ECUDA = 2,         /* a CUDA call failed; see evtb_last_error() */
  EVTB_ENOTFOUND = 3,     /* kernel image or entry point missing */
  EVTB_ENODRIVER = 4,     /* no CUDA driver / device in this process */
  EVTB_EDEVICE_TIMEOUT = 5, /* a bounded device-side wait ran out (status word != 0) */
  EVTB_ETOOLARGE = 6       /* problem exceeds a fixed built-in limit (see evtb_colsum_static) */
};

enum evtb_kind {
  EVTB_GEMM = 0,            /* D = epilogue(A[M,K] x B[K,N])                 FusedGEMM       evt_fuser.py:453 */
  EVTB_BGEMM = 1,           /* batched, operand permutes folded in strides   FusedBMM        evt_fuser.py:561 */
  EVTB_SOFTMAX = 2,         /*                                               FusedSoftmax    evt_fuser.py:700 */
  EVTB_SOFTMAX_BWD = 3,     /*                                               FusedSoftmaxBackward   :765 */
  EVTB_LAYERNORM = 4,       /*                                               FusedLayerNorm         :829 */
  EVTB_LAYERNORM_BWD = 5,   /*                                               FusedLayerNormBackward :905 */
  EVTB_SPMM = 6,            /* CSR SpMM: operands [crow, col, val|0, dinv|0, X]; M = rows, N = F, K = nnz,
                               tile_n = padded F, rows_per_cta = longest row (in nonzeros) that a lane group
                               handles alone (0: 64), stages = nonzeros per task of the longer rows (0: 1024).
                               X must be 32-byte aligned for fp32 features.        FusedSpmm   :973 */
  EVTB_CONV_FPROP = 7,      /* NHWC implicit GEMM: operands [x (N,H,W,C), w (K,R,S,C)], result rows = N*P*Q,
                               columns = K; geometry in evtb_desc.conv         FusedConvFprop  evt_fuser.py:282 */
  EVTB_CONV_DGRAD = 8,      /* data gradient: operands [dy (N,P,Q,K), w (K,R,S,C)], result rows = N*H*W,
                               columns = C                                     FusedConvDgrad  evt_fuser.py:365 */
  EVTB_CONV_WGRAD = 9       /* weight gradient: operands [dy (N,P,Q,K), x (N,H,W,C)], result = the [K, R*S*C]
                               matrix of the channels-last filter gradient; M = K, N = R*S*C, tile_n divides C,
                               split_k cuts the N*P*Q reduction.  In the reference this leaf is a cuDNN call
                               without epilogue (pass_decomposition.py:92-107); here it is an implicit GEMM on
                               the same kernels as the other two passes. */
};

enum evtb_dtype { EVTB_F16 = 0, EVTB_BF16 = 1, EVTB_F32 = 2 };
enum evtb_major { EVTB_MAJOR_K = 0, EVTB_MAJOR_MN = 1 };

/* One GEMM operand as the TMA descriptor needs it (strides in elements). */
typedef struct evtb_matrix {
  int32_t major;          /* evtb_major: which logical dim is contiguous */
  int64_t stride_outer;   /* stride of the other matrix dim */
  int64_t stride_batch;   /* stride between batches (ignored when L == 1) */
} evtb_matrix;

/* Convolution geometry (the reference's Conv2DProblemSize, evt_fuser.py:305-311): x is N x H x W x C,
 * the filter K x R x S x C, the output N x P x Q x K, all channels-last and contiguous; groups = 1. */
typedef struct evtb_conv {
  int32_t N, H, W, C, K, R, S, P, Q;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  /* Forward and weight gradient only: element strides of x between neighbours in w, h and n when x is
   * a strided view instead of a contiguous N x H x W x C tensor (channels always have stride 1); all
   * three 0 = contiguous.  Each must be a multiple of 8 elements (16 bytes).  The strides may describe
   * overlapping windows: a few-channel image seen as N x H x Q x 64 with x_stride_w = stride * channels
   * turns the filter taps of one row into the 64 "channels" the kernels move at a time, which is how
   * the 7 x 7 stem of a ResNet (python/model_zoo/resnet/resnet_modeling.py:190) runs here. */
  int64_t x_stride_w, x_stride_h, x_stride_n;
} evtb_conv;

/* A result tensor that the generated GEMM epilogue writes with TMA bulk stores: element
 * (l, m, n) of the L x M x N result lives at ptr[slot] + l*stride_batch + m*stride_row + n
 * (16-bit elements; strides in elements, multiples of 8).  Listed by the code generator in the
 * order of the epilogue's tensor-map slots. */
typedef struct evtb_tma_store {
  int32_t slot;           /* epilogue pointer slot (index after the main operands) */
  int64_t stride_row;
  int64_t stride_batch;
} evtb_tma_store;

typedef struct evtb_desc {
  int32_t kind;           /* evtb_kind */
  int32_t dtype;          /* evtb_dtype of the main operands */
  int64_t M, N, K, L;     /* GEMM: problem; reduce-apply: M = rows, N = columns, K = L = 1 */
  evtb_matrix a, b;       /* GEMM / BGEMM only */
  int32_t tile_n;         /* GEMM: accumulator tile is 128 x tile_n */
  int32_t stages;         /* GEMM: depth of the shared-memory ring */
  int32_t threads;        /* CTA size of the generated kernel */
  int32_t smem_bytes;     /* dynamic shared memory of the generated kernel */
  int32_t rows_per_cta;   /* reduce-apply: rows one CTA owns per step */
  int32_t n_epilogue_ptrs;/* pointer slots of the generated epilogue (after the main operands) */
  const char* image_path; /* cubin produced by the code generator */
  const char* entry;      /* kernel name inside the image */
  int32_t sm_count;       /* 0 = ask the device */
  int32_t split_k;        /* GEMM: cut K into this many units per tile (<= 1: off).  The image must be
                             generated for split-K; the plan then needs a workspace. */
  int32_t cta_pair;       /* GEMM: 1 = the image is the CTA-pair variant (cluster of two CTAs, 256 x tile_n
                             output tile, tile_n 128 or 256; with split_k each CTA parks the partial of its
                             own 128-row half); the grid is sized to the number of clusters the device can
                             hold at once. */
  int32_t row_resident;   /* GEMM / BGEMM: 1 = the image is the row-resident variant (128 x 512 accumulator tile,
                             N <= 512, tile_n = 512): a row-wise softmax / softmax-backward step of the
                             epilogue runs over whole rows held in tensor memory.  No reference counterpart
                             (there the step is a separate kernel, evt_fuser.py:700-826). */
  int32_t n_tma_stores;   /* GEMM / BGEMM: results written through TMA (0..4) */
  evtb_tma_store tma_stores[4];
  evtb_conv conv;         /* CONV_* only.  Channel counts must be multiples of 64 (operands move in 64-channel
                             blocks through TMA boxes), dilation 1 for the data gradient. */
} evtb_desc;

/* Per-launch scalars (all optional; pass NULL for none). */
typedef struct evtb_scalars {
  float scalar[8];
  uint64_t seed;          /* fused-dropout RNG (Philox) */
  uint64_t rng_offset;
} evtb_scalars;

int evtb_version(void);
const char* evtb_status_string(int status);
const char* evtb_last_error(void);

int evtb_plan_create(const evtb_desc* desc, evtb_plan** out);
int evtb_plan_destroy(evtb_plan* plan);
/* Scratch the caller must provide to evtb_launch (0 for most plans; split-K GEMMs keep their
 * fp32 partial tiles and per-tile arrival counters there, SpMM plans the task list and the
 * partial sums of their long rows).  It must be 16-byte aligned and
 * ZERO-FILLED once before its first use; launches leave it ready for the next one.  Launches
 * that share a workspace must be ordered on one stream. */
int evtb_plan_workspace_bytes(const evtb_plan* plan, size_t* bytes);
/* Number of main operands that precede the epilogue pointers in `operand_ptrs`. */
int evtb_plan_num_main_operands(const evtb_plan* plan, int* n);
/* CTAs the plan launches (for reporting). */
int evtb_plan_grid(const evtb_plan* plan, int* ctas);

/* operand_ptrs = [main operands..., epilogue slot 0, slot 1, ...]; n = their count.
 * status_word: device int the kernel writes a non-zero code to if a bounded wait ran out
 * (may be NULL).  Enqueues only. */
int evtb_launch(evtb_plan* plan, const void* const* operand_ptrs, int n, void* workspace,
                void* status_word, evtb_stream stream);
/* Diagnostic, no reference counterpart: kernels compiled with -DEVTB_PROFILE write eight
 * clock64 counters per CTA (kernel, producer wait, MMA data wait, MMA accumulator wait, epilogue
 * wait, epilogue work, 2 spare) to `device_buffer` (grid x 8 x int64).  Ignored by other kernels. */
int evtb_plan_set_profile_buffer(evtb_plan* plan, void* device_buffer);

int evtb_launch_ex(evtb_plan* plan, const void* const* operand_ptrs, int n, void* workspace,
                   void* status_word, evtb_stream stream, const evtb_scalars* scalars);

/* y[c] = sum over rows of x[rows, cols] (row-major, contiguous), accumulated in fp32 in a fixed
 * order, written in `out_dtype`.  Bias gradients whose producer is a row kernel rather than a
 * GEMM use this; in the reference such `aten.sum` nodes are left to eager / TorchScript
 * (python/gtl/compiler/passes/evt_fuser.py:1096-1100, nv_fuser.py:134-141).
 * `workspace`: evtb_colsum_workspace_bytes() bytes, 16-byte aligned, ZERO-FILLED once before
 * its first use (the kernel leaves it ready for the next call).  Calls that share one
 * workspace must be ordered on one stream. */
/* y[c] += sum over rows of x[rows, cols], y fp32: one pass with fp32 atomics (order of additions not
 * fixed), no workspace.  y must hold the value to add to -- zero for a plain sum; callers that carve
 * many such targets from one pre-zeroed buffer pay one memset for all of them. */
int evtb_colsum_accumulate(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, float* y, evtb_stream stream);
int evtb_colsum_workspace_bytes(int64_t rows, int64_t cols, size_t* bytes);
int evtb_colsum(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, void* y, int32_t out_dtype,
                void* workspace, size_t workspace_bytes, evtb_stream stream);

/* Training-mode batch norm on a channels-last activation seen as [rows, channels] (rows = N*H*W,
 * fp16 or bf16, contiguous, 16-byte aligned, channels % 8 == 0, channels <= 4096): the three leaves the
 * reference's decomposition leaves outside a convolution epilogue -- batch_norm_elemt,
 * batch_norm_backward_stat, batch_norm_backward_elemt
 * (python/gtl/compiler/passes/pass_decomposition.py:143-189) -- one pass over the activation each.
 * Per-channel statistics are fp32 vectors; gamma / beta / dgamma / dbeta have the activation's type.
 * Nothing is allocated; enqueue only.
 *
 * evtb_bn_apply: z = (y - mean) * rstd * gamma + beta, rstd = rsqrt(mean_sq - mean^2 + eps), from the
 *   E[y], E[y^2] vectors a convolution epilogue produced; optionally + residual (NULL for none) and
 *   max(., 0) (relu != 0).  saved_mean / saved_rstd (NULL to skip) receive the statistics.
 * evtb_bn_backward_reduce: g' = grad (+ grad2 if not NULL) (zeroed where act <= 0 if act is not NULL),
 *   written to grad_out (required when g' differs from grad, else may be NULL);
 *   sums[c] += sum_r g'[r, c], sums[channels + c] += sum_r g'[r, c] * (y[r, c] - mean[c]) * rstd[c]
 *   with fp32 atomics: the caller zero-fills `sums` (2 * channels floats) before the launch.
 * evtb_bn_backward_apply: dy = (grad - sums[c] * rf - x_hat * sums[channels + c] * rf) * gamma * rstd;
 *   dgamma = sums[channels + c], dbeta = sums[c] (NULL to skip). */
int evtb_bn_apply(const void* y, int32_t dtype, int64_t rows, int64_t channels, const float* mean, const float* mean_sq,
                  const void* gamma, const void* beta, float eps, const void* residual, int32_t relu, void* z,
                  float* saved_mean, float* saved_rstd, evtb_stream stream);
int evtb_bn_backward_reduce(const void* grad, const void* grad2, const void* act, const void* y, int32_t dtype,
                            int64_t rows, int64_t channels, const float* mean, const float* rstd, void* grad_out,
                            float* sums, evtb_stream stream);
int evtb_bn_backward_apply(const void* grad, const void* y, int32_t dtype, int64_t rows, int64_t channels,
                           const float* mean, const float* rstd, const void* gamma, const float* sums,
                           float reduction_factor, void* dy, void* dgamma, void* dbeta, evtb_stream stream);

/* Max-pooling of a channels-last activation x [N, H, W, C] (fp16 / bf16, contiguous, C % 8 == 0), square
 * window `kernel` <= 15, `stride`, zero-free padding `padding` (padded positions never win), floor mode,
 * dilation 1: the reference's leaves max_pool2d_with_indices_channel_last and
 * max_pool2d_with_indices_backward_channel_last (python/gtl/compiler/passes/pass_decomposition.py:109-132).
 * Instead of the library's int64 index per output element, `code` holds one byte per output element:
 * r * kernel + t, the place of the maximum inside its window (first maximum in scan order, a NaN wins --
 * the library's rule).  y and code have N x P x Q x C elements, P = (H + 2 padding - kernel) / stride + 1.
 * Backward: dx[n, h, w, c] = sum of dy over the windows that cover (h, w) and chose it. */
int evtb_maxpool_forward(const void* x, int32_t dtype, int64_t N, int64_t H, int64_t W, int64_t C, int32_t kernel,
                         int32_t stride, int32_t padding, void* y, uint8_t* code, evtb_stream stream);
int evtb_maxpool_backward(const void* dy, const uint8_t* code, int32_t dtype, int64_t N, int64_t H, int64_t W, int64_t C,
                          int32_t kernel, int32_t stride, int32_t padding, void* dx, evtb_stream stream);

/* SDDMM on a CSR pattern (int32 indices, fp32 features, F % 4 == 0):
 * out[p] = dot(U[i, :], V[col[p], :]) for every stored (i, col[p]).  Edge gradients of a GCN
 * layer; the reference has no SDDMM (its GCN backward is a second SpMM,
 * python/model_zoo/gcn/gcn_modeling.py:107-120) -- required by the GCN configuration here. */
int evtb_sddmm(const int32_t* crow, const int32_t* col, const float* u, const float* v, int64_t rows, int64_t nnz,
               int64_t F, float* out, evtb_stream stream);

/* COO -> CSR (int32): sort (row, col) pairs, drop duplicates, find row starts; crow has
 * rows + 1 entries, col has room for n_edges, *nnz_out (device int) receives the count.
 * Replaces the host-side dgl/torch CSR construction of python/model_zoo/gcn/gcn.py:57-66.
 * workspace: evtb_csr_build_workspace_bytes() bytes, 256-byte aligned (no zero-fill needed). */
int evtb_csr_build_workspace_bytes(int64_t n_edges, size_t* bytes);
int evtb_csr_build(const int32_t* coo_row, const int32_t* coo_col, int64_t n_edges, int64_t rows, void* workspace,
                   size_t workspace_bytes, int32_t* crow, int32_t* col, int32_t* nnz_out, evtb_stream stream);

/* evtb_colsum for hosts that cannot provide scratch memory.  (No counterpart in the reference:
 * its runtime always allocates through torch.)  Meant for callers such as a serving process
 * that handed its entire device-memory budget to its own pool at start-up, or a plugin slot
 * where a cudaMalloc -- which synchronises the whole device -- must not happen.  The partial
 * sums live in an array built into the library image (about 2 MiB on every GPU that loads the
 * library, held until the process exits), so:
 *   - cols is limited to evtb_colsum_static_max_cols() (8192); larger problems return
 *     EVTB_ETOOLARGE and launch nothing;
 *   - this function and everything it calls allocates nothing (no cudaMalloc / cudaFree, no
 *     torch allocation); inputs and outputs are still the caller's;
 *   - every call uses the array of the CURRENT device: make the device that owns x, y and the
 *     stream current before calling (a buffer of another device is refused with EVTB_EINVAL);
 *     the first call on each device looks the array's device address up (a host-side CUDA
 *     query); make that first call outside any stream capture;
 *   - all calls share the one array: calls whose kernels may overlap on the GPU (different
 *     streams, no ordering between them) race and give wrong sums.  Order them. */
int evtb_colsum_static_max_cols(void);
int evtb_colsum_static(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, void* y, int32_t out_dtype,
                       evtb_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* EVT_B200_H_ */
