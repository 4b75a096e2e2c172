/* ss2d_b200 -- C ABI of the B200 (sm_100a) SS2D core library, libss2d_b200.so.
 *
 * Plain C types only: raw device pointers, sizes and strides in ELEMENTS (int64),
 * a CUDA stream passed as an opaque pointer.  The library never allocates, frees or
 * retains memory: the caller owns every buffer (inputs, outputs, workspace), inputs are
 * read-only, outputs are fully overwritten.  Every entry point validates its arguments
 * before launching anything, launches asynchronously on the given stream, never
 * synchronises, and returns 0 or a negative ss2d_status.  No exception crosses the ABI.
 *
 * File names cited below are paths inside MzeroMiko/VMamba.
 */
#ifndef SS2D_B200_H
#define SS2D_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SS2D_ABI_VERSION 1
#define SS2D_ROUTES 4            /* K: the four scan routes of SS2D */
#define SS2D_MAX_DSTATE 256      /* as kernels/selective_scan/cusoflex/selective_scan_oflex.cpp:180 */

typedef enum ss2d_dtype { SS2D_F32 = 0, SS2D_F16 = 1, SS2D_BF16 = 2 } ss2d_dtype;

typedef enum ss2d_status {
    SS2D_OK = 0,
    SS2D_EINVAL_NULL = -1,     /* a required pointer is NULL */
    SS2D_EINVAL_SHAPE = -2,    /* a size is zero/negative or sizes disagree */
    SS2D_EINVAL_DTYPE = -3,    /* unknown or unsupported dtype combination */
    SS2D_EINVAL_ALIGN = -4,    /* a pointer is not aligned to its element size */
    SS2D_EINVAL_STRIDE = -5,   /* a stride is impossible for the given sizes */
    SS2D_ENOTSUP = -6,         /* valid request that this build does not implement */
    SS2D_ECUDA = -7,           /* the CUDA runtime reported an error at launch */
    SS2D_EWORKSPACE = -8,      /* workspace missing or too small */
    SS2D_ETOOBIG = -9,         /* problem exceeds the built-in scratch of an allocation-free entry point */
    SS2D_EINVAL_DEVICE = -10   /* debug checks on: a pointer is host memory or belongs to another GPU than the current one */
} ss2d_status;

/* ------------------------------------------------------------------------------------
 * Selective-scan forward.  Replaces selective_scan_cuda_oflex.fwd
 * (kernels/selective_scan/cusoflex/selective_scan_oflex.cpp:143-231, kernel
 * cusoflex/selective_scan_fwd_kernel_oflex.cuh:67-181) as called by SelectiveScanCuda.forward
 * (classification/models/csms6s.py:74-87, vmamba.py:840-853); same mathematics as
 * selective_scan_torch (csms6s.py:25-68).
 *
 * For every row (b, r), r in [0, dim), group k = r / (dim / n_groups), state h in R^dstate = 0:
 *   dl   = delta[b, r, l] (+ delta_bias[r]) ; dl = softplus(dl) if delta_softplus
 *   h_n  = exp(dl * A[r, n]) * h_n + dl * B[b, k, n, l] * u[b, r, l]
 *   out[b, r, l] = sum_n C[b, k, n, l] * h_n (+ D[r] * u[b, r, l])
 * u, delta, out: (batch, dim, seqlen), last dimension contiguous, strides in elements.
 * A: (dim, dstate) fp32 contiguous.  B, C: (batch, n_groups, dstate, seqlen), last dimension
 * contiguous.  D, delta_bias: (dim) fp32 or NULL.  in_dtype is the type of u, delta, B, C;
 * out_dtype is SS2D_F32 ("oflex") or equal to in_dtype.  State and arithmetic are fp32.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_scan_params {
    const void *u, *delta, *A, *B, *C, *D, *delta_bias;
    void *out;
    int32_t in_dtype, out_dtype;
    int32_t delta_softplus;
    int32_t delta_ratio;                /* channels sharing one delta row (and one delta_bias entry): delta is
                                           (batch, dim / delta_ratio, seqlen), row r / delta_ratio serves channel r
                                           (selective_scan_oflex.cpp:59, 176-183); 0 or 1 = one row per channel */
    int64_t batch, dim, dstate, seqlen, n_groups;
    int64_t u_batch_stride, u_dim_stride;
    int64_t delta_batch_stride, delta_dim_stride;
    int64_t out_batch_stride, out_dim_stride;
    int64_t B_batch_stride, B_group_stride, B_state_stride;
    int64_t C_batch_stride, C_group_stride, C_state_stride;
    void *checkpoints;                  /* optional, fp32 (batch, dim, ceil(seqlen / 128), dstate) contiguous: the state
                                           in front of every 128th element, for ss2d_selective_scan_bwd (the reference
                                           hands its backward the chunk states `x` the same way, selective_scan_oflex.cpp:208) */
} ss2d_scan_params;

int ss2d_selective_scan_fwd(const ss2d_scan_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * Selective-scan backward.  Replaces selective_scan_cuda_oflex.bwd
 * (kernels/selective_scan/cusoflex/selective_scan_oflex.cpp:233-355, kernel
 * cusoflex/selective_scan_bwd_kernel_oflex.cuh:73-290) as called by SelectiveScanCuda.backward
 * (classification/models/csms6s.py:89-109); same gradients as autograd through
 * selective_scan_torch (csms6s.py:25-68).
 *
 * Inputs as in the forward call plus dout (batch, dim, seqlen) of dout_dtype (SS2D_F32 or
 * in_dtype), last dimension contiguous.  Nothing saved by the forward call is needed: the states
 * are recomputed.  Results (all fully overwritten, all contiguous):
 *   du, ddelta (batch, dim, seqlen) in_dtype;  dA (dim, dstate) fp32;
 *   dB, dC (batch, n_groups, dstate, seqlen) in_dtype, summed in fp32 over the channels of a group;
 *   dD, ddelta_bias (dim) fp32, required exactly when D / delta_bias is given.
 * workspace: ss2d_selective_scan_bwd_workspace_bytes() bytes, 16-byte aligned (fp32 partial sums).
 * No atomics: repeated calls give bit-identical results.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_scan_bwd_params {
    const void *u, *delta, *A, *B, *C, *D, *delta_bias;
    const void *dout;
    void *du, *ddelta, *dA, *dB, *dC, *dD, *ddelta_bias;
    void *workspace;
    int64_t workspace_bytes;
    int32_t in_dtype, dout_dtype;
    int32_t delta_softplus;
    int32_t delta_ratio;                /* as in ss2d_scan_params; ddelta is still written per channel (batch, dim, seqlen)
                                           and ddelta_bias per channel (dim): the caller sums the delta_ratio rows that
                                           share an input row, as selective_scan_oflex.cpp:348-352 does */
    int64_t batch, dim, dstate, seqlen, n_groups;
    int64_t u_batch_stride, u_dim_stride;
    int64_t delta_batch_stride, delta_dim_stride;
    int64_t dout_batch_stride, dout_dim_stride;
    int64_t B_batch_stride, B_group_stride, B_state_stride;
    int64_t C_batch_stride, C_group_stride, C_state_stride;
    const void *checkpoints;            /* optional: what the forward call wrote; saves the pass that recomputes the states */
} ss2d_scan_bwd_params;

int64_t ss2d_selective_scan_bwd_workspace_bytes(const ss2d_scan_bwd_params *p);   /* < 0: invalid or unsupported arguments */
int ss2d_selective_scan_bwd(const ss2d_scan_bwd_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * CrossScan / CrossMerge, channel-first tensors.  Replace CrossScanTritonF.forward and
 * CrossMergeTritonF.forward / triton_cross_scan_flex (classification/models/csm_triton.py:
 * 278-497; vmamba.py:350-575) and compute exactly cross_scan_fwd / cross_merge_fwd
 * (vmamba.py:41-130): pure data movement, bit-exact.
 *   scan : x (B, C, H, W)      -> xs (B, 4, C, H*W)
 *   merge: ys (B, 4, C, H, W)  -> y  (B, C, H*W), summed in the reference's association order
 * scans: 0 cross (row-major, column-major, both reversed), 1 unidirectional, 2 bidirectional,
 * 3 rotations by 90 degrees.  All tensors contiguous.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_cross_params {
    const void *in;
    void *out;
    int32_t dtype;
    int32_t scans;
    int64_t B, C, H, W;
} ss2d_cross_params;

int ss2d_cross_scan(const ss2d_cross_params *p, void *cuda_stream);
int ss2d_cross_merge(const ss2d_cross_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * CrossScan / CrossMerge with the reference's layout flags (cross_scan_fwd / cross_merge_fwd / their one-by-one
 * forms, vmamba.py:41-245; CrossScanF / CrossMergeF, csm_triton.py:182-273).  In both calls in_channel_first names
 * the layout of the map side ((B, C, H, W) or (B, H, W, C)) and out_channel_first the layout of the routes side
 * ((B, 4, C, L) or (B, L, 4, C)), as in the reference.
 *   ss2d_cross_scan_ex : map -> routes;  one_by_one: in is (B, 4, C, H, W) or, channel-last, (B, H, W, 4, C), and
 *                        route k reads its own map
 *   ss2d_cross_merge_ex: routes -> map (B, C, L) or (B, L, C);  one_by_one: no sum, out is (B, 4, C, L) or, with
 *                        in_channel_first 0, (B, L, 4, C)
 * one_by_one with channel-first tensors on both sides takes scans 0-3; with a channel-last side it takes scans 0-2,
 * the route sets the reference's GPU kernel defines (csm_triton.py:313-336), and returns SS2D_ENOTSUP for 3.  With
 * scans 1 the four maps pass through in row-major order.  Index-only variants, not tuned.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_cross_ex_params {
    const void *in;
    void *out;
    int32_t dtype;
    int32_t scans;
    int32_t in_channel_first, out_channel_first, one_by_one, reserved0;
    int64_t B, C, H, W;
} ss2d_cross_ex_params;

int ss2d_cross_scan_ex(const ss2d_cross_ex_params *p, void *cuda_stream);
int ss2d_cross_merge_ex(const ss2d_cross_ex_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * Fused SS2D core: CrossScan folded into the scan's loads + four-route selective scan
 * (d_state >= 1) + CrossMerge + LayerNorm over channels, for scans mode 0.  Replaces the
 * chain cross_scan_fn -> selective_scan_fn -> cross_merge_fn -> out_norm -> cast of
 * SS2Dv2.forward_corev2 (vmamba.py:1536, 1553-1557, 1566-1571); the (B, 4, D, L) copy of x
 * and the per-route outputs never exist in memory.
 *
 *   x        (B, D, H, W), act_dtype; planes contiguous, batch / channel strides given (see below)
 *   delta[k] (B, D, L) per route k, act_dtype, contiguous planes (batch stride given), raw
 *            (pre-bias, pre-softplus) step sizes, stored in the ORIENTATION ORDER of route k:
 *            index h*W+w for k = 0, 2 and w*H+h for k = 1, 3 (never reversed)
 *   Bm[k], Cm[k] (B, N, L) per route, same order, act_dtype (the type the projection produced them in,
 *            as the reference's Bs / Cs are: selective_scan_oflex.cpp:157-159)
 *   A (4*D, N), Dskip (4*D), delta_bias (4*D): fp32, row index k*D + d
 *   ln_weight, ln_bias (D) fp32 or NULL (NULL: no affine); ln_eps; with_norm = 0 skips LayerNorm
 *   y        (B, D, H, W), y_dtype (act_dtype or SS2D_F32), own batch / channel strides
 *   workspace: ss2d_core_workspace_bytes() bytes, 256-byte aligned (holds the fp32 merged map)
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_core_params {
    const void *x;
    const void *delta[SS2D_ROUTES];
    const void *Bm[SS2D_ROUTES];
    const void *Cm[SS2D_ROUTES];
    const void *A, *Dskip, *delta_bias;
    const void *ln_weight, *ln_bias;
    void *y;
    void *workspace;
    int64_t workspace_bytes;
    int64_t delta_batch_stride[SS2D_ROUTES];
    int64_t bc_batch_stride[SS2D_ROUTES];
    int64_t B, D, H, W, N;
    int32_t act_dtype, y_dtype;
    int32_t with_norm;
    float ln_eps;
    /* layout of x and of y: element strides between images and between channels; pixels of one
     * (image, channel) plane are always contiguous.  0 = dense channel-first (D*L and L).
     * (D, B, H, W) "channel-major" maps are batch stride L, channel stride B*L. */
    int64_t x_batch_stride, x_channel_stride;
    int64_t y_batch_stride, y_channel_stride;
    int64_t delta_channel_stride[SS2D_ROUTES];   /* 0 = L; (D, B, L) step-size maps: L as batch stride and B*L here */
} ss2d_core_params;

int64_t ss2d_core_workspace_bytes(const ss2d_core_params *p);
int ss2d_core_fwd(const ss2d_core_params *p, void *cuda_stream);
/* SS2D_OK when ss2d_core_fwd takes this problem itself (d_state 1, a plane that fits one CTA with the
 * given alignments and strides), otherwise the status ss2d_core_fwd would return before launching
 * anything (SS2D_ENOTSUP: use the operator-surface kernels).  Reads sizes, dtypes, strides and the
 * alignment of the pointers only; the workspace fields are ignored and nothing is dereferenced.  Takes the
 * place of the shape tests of selective_scan_fwd (selective_scan_oflex.cpp:152-204) for the fused call. */
int ss2d_core_supported(const ss2d_core_params *p);

/* ------------------------------------------------------------------------------------
 * Elementwise producers around the core, channel-first (B, D, H, W) contiguous maps of `dtype`.
 *   ss2d_bias_act:      y = act(x + bias[d]); x and y may be the same buffer.  Replaces the bias
 *                       addition and activation of Mlp.forward (vmamba.py:1160-1163).
 *   ss2d_dwconv3x3_act: y = act(depthwise 3x3 convolution of x, stride 1, zero padding 1,
 *                       weight (D, 3, 3) of `dtype`, optional fp32 bias).  Replaces
 *                       self.conv2d followed by self.act in SS2Dv2.forwardv2 (vmamba.py:1582-1583).
 * act: 0 none, 1 GELU (erf form), 2 SiLU.  Sums are formed in fp32, rounded to `dtype`, then the
 * activation is applied and rounded, like the separate kernels these calls replace.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_pointwise_params {
    const void *x;
    const void *weight;     /* dwconv only */
    const void *bias;       /* (D) fp32 or NULL */
    void *y;
    int64_t B, D, H, W;
    int32_t dtype, act;
    int32_t channel_major;   /* 0: maps are (B, D, H, W); 1: (D, B, H, W) */
    int32_t reserved0;
} ss2d_pointwise_params;

int ss2d_bias_act(const ss2d_pointwise_params *p, void *cuda_stream);
int ss2d_dwconv3x3_act(const ss2d_pointwise_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * Route expansion: from x_dbl = x_proj(x), computed once on the map in its native pixel order, to
 * the per-route streams ss2d_core_fwd consumes.  Replaces, for scans mode 0, the dt_projs grouped
 * 1x1 convolution, the split and the three .contiguous() copies of SS2Dv2.forward_corev2
 * (vmamba.py:1538-1543, 1546-1547), applied to projections of the un-scanned map (a 1x1 projection
 * commutes with the CrossScan permutation, vmamba.py:1536-1537).
 *   x_dbl     (B, 4, R+2N, L) act_dtype, pixel order h*W+w; strides in elements for batch, route and row
 *             (a GEMM on a channel-major map yields (4, R+2N, B, L): batch L, route (R+2N)*B*L, row B*L)
 *   dt_weight (4, D, R) act_dtype contiguous (dt_projs.weight viewed per route)
 *   delta[k]  (B, D, L) act_dtype  = dt_weight[k] . x_dbl[:, k, :R]  in the orientation order of route k
 *   bc[k]     (B, 2N, L) act_dtype = x_dbl[:, k, R:] (B rows then C rows) in the same order
 * 16-bit maps with R > 12 run the contraction on the tensor cores (mma.sync, fp32 accumulation); the result is
 * rounded to act_dtype once, like the library GEMM this replaces.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_expand_params {
    const void *x_dbl;
    const void *dt_weight;
    void *delta[SS2D_ROUTES];
    void *bc[SS2D_ROUTES];
    int64_t x_dbl_batch_stride, x_dbl_route_stride;
    int64_t x_dbl_row_stride;           /* between projected rows; 0 = L (dense (B, 4, R+2N, L)) */
    int64_t delta_batch_stride[SS2D_ROUTES];
    int64_t bc_batch_stride[SS2D_ROUTES];
    int64_t delta_channel_stride[SS2D_ROUTES];   /* 0 = L; (D, B, L) outputs: batch stride L, channel stride B*L */
    int64_t bc_row_stride[SS2D_ROUTES];          /* 0 = L; (2N, B, L) outputs: batch stride L, row stride B*L */
    int64_t B, D, R, N, H, W;
    int32_t act_dtype;
    int32_t reserved0;
    void *workspace;                    /* optional: ss2d_route_expand_workspace_bytes() bytes, 16-byte aligned */
    int64_t workspace_bytes;
} ss2d_expand_params;

/* With a workspace the projected rows of the two column-major routes are transposed once, plane by plane, by a
 * small kernel in front (2 * (R+2N) * B * H * W elements), and the expansion reads every route contiguously;
 * without one (NULL) it gathers them with strided 2-byte loads, which costs about a third more time. */
int64_t ss2d_route_expand_workspace_bytes(const ss2d_expand_params *p);

int ss2d_route_expand(const ss2d_expand_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * Fused MLP of a VSS block on a channel-major map:  y = W2 . gelu(W1 . x + b1), erf-form GELU, the
 * hidden activations (4C per pixel) kept on chip.  Replaces fc1, the activation and fc2 of
 * Mlp.forward (vmamba.py:1151-1167, channel-first form :1060-1064); the fc2 bias is NOT added
 * (ss2d_layer_norm_cf adds it with the residual update, as `add_bias`).
 *   x  (C, N)  dtype (SS2D_BF16 or SS2D_F16), N = B*H*W pixels contiguous per channel, N % 8 == 0
 *   w1 (hidden, C) dtype, row-major; b1 (hidden) fp32; w2 (C, hidden) dtype, row-major
 *   y  (C, N)  dtype
 * Runs on the tcgen05 tensor cores (fp32 accumulation in tensor memory), operands staged by TMA.
 * ss2d_mlp_supported returns SS2D_OK when ss2d_mlp_fwd takes the problem (hidden == 4 C and a width
 * whose weights fit one SM: C == 96), else the status ss2d_mlp_fwd would return without launching
 * (SS2D_ENOTSUP: use two GEMMs and ss2d_bias_act).
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_mlp_params {
    const void *x;
    const void *w1;
    const void *b1;
    const void *w2;
    void *y;
    int64_t C, hidden, N;
    int32_t dtype;
    int32_t reserved0;
} ss2d_mlp_params;

int ss2d_mlp_supported(const ss2d_mlp_params *p);
int ss2d_mlp_fwd(const ss2d_mlp_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * 1x1 projection of a channel-major map:  out (M, N) = w (M, K) . x (K, N) (+ bias[m]), N = B*H*W pixels
 * contiguous in every row.  With the stacked x_proj weights of the four routes as w ((4 (R + 2N), D)) this is
 * the x_proj contraction of forward_corev2 (vmamba.py:1536-1538: a grouped conv1d on the (B, 4 D, L) scan copy)
 * computed on the un-scanned map, which a 1x1 projection permits; with a bias it is Linear2d.forward
 * (vmamba.py:1062-1075).
 *   x   (K, N)  dtype (SS2D_BF16 or SS2D_F16), rows x_row_stride elements apart (0 = N; a multiple of 8)
 *   w   (M, K)  dtype, row-major, M <= 256, K a multiple of 32
 *   bias (M) fp32 or NULL;   out (M, N) dtype, rows out_row_stride elements apart (0 = N)
 * Runs on the tcgen05 tensor cores (fp32 accumulation in tensor memory), operands staged by TMA.
 * ss2d_linear_supported returns SS2D_OK when ss2d_linear_fwd takes the problem, else the status it would
 * return without launching (SS2D_ENOTSUP: use a library GEMM).
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_linear_params {
    const void *x;
    const void *w;
    const void *bias;
    void *out;
    int64_t M, K, N;
    int64_t x_row_stride, out_row_stride;
    int32_t dtype;
    int32_t reserved0;
} ss2d_linear_params;

int ss2d_linear_supported(const ss2d_linear_params *p);
int ss2d_linear_fwd(const ss2d_linear_params *p, void *cuda_stream);

/* Debug checks (off by default; on with the environment variable SS2D_DEBUG_CHECKS=1 at load time or by this call).
 * When on, every entry point that launches kernels first asks the driver about each pointer it was given
 * (cudaPointerGetAttributes) and returns SS2D_EINVAL_DEVICE, before any launch, for host memory or memory of a GPU
 * other than the current one - the consistency the reference gets from its tensor checks (u.is_cuda() and same-device
 * guards, selective_scan_oflex.cpp:152-204).  Costs a driver call per pointer, hence the switch.  Returns the old state. */
int ss2d_set_debug_checks(int on);

/* Allocation-free form of ss2d_core_fwd.  It has no counterpart in the reference: it exists for
 * callers that can hand over inputs and outputs but cannot obtain device memory themselves (an
 * operator slot of a serving runtime that passes only pre-placed tensors, a host language bound to
 * this ABI without a CUDA allocator, a process whose device memory is fixed at start-up).  The
 * fp32 scratch map that ss2d_core_fwd takes as `workspace` lives in a static device array inside
 * the library instead (32 MiB on every GPU that loads the library, held until the process ends);
 * `workspace` / `workspace_bytes` of the params are ignored.
 *   - limit: B*D*H*W <= ss2d_core_static_capacity() (8 388 608); beyond it the call returns
 *     SS2D_ETOOBIG and launches nothing;
 *   - the first call on a device resolves the device address of that array; issue it outside
 *     any stream capture;
 *   - calls on the same GPU share the array and must not overlap in time (they would race);
 *     nothing in it needs clearing between calls;
 *   - never calls cudaMalloc/cudaFree.  Results are identical to ss2d_core_fwd's. */
int ss2d_core_fwd_static(const ss2d_core_params *p, void *cuda_stream);
int64_t ss2d_core_static_capacity(void);

/* LayerNorm over the channel axis of a channel-first map with an optional fused residual update:
 *   s = in (+ add) (+ add_bias[d]);  sum_out = s (if given);  out = LN_D(s) * weight + bias.
 * Replaces LayerNorm(channel_first=True).forward (vmamba.py:1087-1093) + the trailing cast
 * (vmamba.py:1571) and, with `add`, the residual additions of VSSBlock._forward
 * (vmamba.py:1772, 1777) together with the norm that follows them.
 *   in       (B, D, L) fp32 or NULL  add      (B, D, L) io_dtype or NULL (at least one of the two)
 *   add_bias (D) fp32 or NULL        sum_out  (B, D, L) fp32 or NULL; may be the same buffer as `in`
 *   weight, bias (D) fp32 or NULL    out      (B, D, L) io_dtype
 * Pixels of a plane are contiguous; `channel_stride` and `batch_stride` in elements (0 = dense
 * channel-first: L and D*L).  `out` may use a different pair, which converts between the
 * (B, D, L) and (D, B, L) layouts on the way. */
typedef struct ss2d_norm_params {
    const void *in;
    const void *add;
    const void *add_bias;
    void *sum_out;
    const void *weight, *bias;
    void *out;
    int64_t B, D, L;
    int64_t batch_stride, channel_stride;           /* of in, add, sum_out */
    int64_t out_batch_stride, out_channel_stride;   /* of out; 0 = same as the inputs */
    int32_t io_dtype;
    float eps;
    int32_t skip_norm;      /* 1: out = s converted to io_dtype, no normalisation (fused add, cast, layout change) */
    int32_t descending;     /* 1: the map is walked from its last image to its first.  Same result; for an `in` that the
                             * kernel before wrote front to back and that is larger than L2, the end is still cached */
} ss2d_norm_params;

int ss2d_layer_norm_cf(const ss2d_norm_params *p, void *cuda_stream);

/* library identification and error text */
/* ------------------------------------------------------------------------------------
 * First layer of the patch embedding, fused: 3x3 convolution, stride 2, padding 1, in_channels 3 -> C0
 * (+ bias), LayerNorm over the C0 channels of each pixel, GELU.  Replaces the first three modules of
 * VSSM._make_patch_embed_v2 (vmamba.py:1928-1942: Conv2d, LayerNorm2d, GELU).
 *   x (B, 3, H, W) dtype, contiguous;  weight (C0, 3, 3, 3) dtype;  conv_bias, ln_weight, ln_bias (C0) fp32 or NULL
 *   y (B, ceil(H/2), ceil(W/2), C0) dtype, PIXEL-MAJOR (channels of a pixel contiguous), 16-byte aligned
 * C0 in {32, 48, 64}, act = 1 (GELU); anything else returns SS2D_ENOTSUP.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_stem_params {
    const void *x, *weight, *conv_bias, *ln_weight, *ln_bias;
    void *y;
    int64_t B, H, W, C0, in_channels;
    int32_t dtype, act;
    float eps;
    int32_t reserved0;
} ss2d_stem_params;

int ss2d_stem_conv_norm_act(const ss2d_stem_params *p, void *cuda_stream);

/* ------------------------------------------------------------------------------------
 * Layout changes between pixel-major rows (N, C) - the layout the library convolutions of the patch
 * embedding and of the downsampling layers run in - and channel planes (C, N), N = all pixels of the
 * batch in (image, row, column) order, with the neighbouring elementwise work folded in.
 *
 * ss2d_pixels_norm_to_planes: planes[c, n] = LayerNorm_c(rows[n, :] + bias)[c]   (the LayerNorm2d after a
 *   strided convolution, vmamba.py:1940, 1969; the convolution's bias joins here).  rows: rows_dtype,
 *   16-byte aligned, C a multiple of 8 (16-bit) or 4 (fp32), C <= 2048 / 1024; planes: SS2D_F32 or rows_dtype.
 * ss2d_planes_to_pixels: v = planes[c, n] (+ add[c, n] + bias[c]); rows[n, c] = v; with sum_out == planes the
 *   fp32 planes are updated in place (the last residual addition of a stage, vmamba.py:1772/1777, in front of
 *   the downsampling convolution).  planes: SS2D_F32; add: rows_dtype, same plane stride.
 * plane_stride: elements between planes, 0 = N.  Fields a call does not use must be NULL.
 * -------------------------------------------------------------------------------- */
typedef struct ss2d_relayout_params {
    void *rows;
    void *planes;
    const void *add, *bias, *ln_weight, *ln_bias;
    void *sum_out;
    int64_t N, C, plane_stride;
    int32_t rows_dtype, planes_dtype;
    float eps;
    int32_t reserved0;
} ss2d_relayout_params;

int ss2d_pixels_norm_to_planes(const ss2d_relayout_params *p, void *cuda_stream);
int ss2d_planes_to_pixels(const ss2d_relayout_params *p, void *cuda_stream);

int ss2d_version(void);
const char *ss2d_strerror(int status);
/* number of kernel launches issued by this library in this process so far (all entry points) */
int64_t ss2d_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SS2D_B200_H */
