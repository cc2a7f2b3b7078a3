/*
 * d2dmoe.h — C ABI of the B200 (sm_100a) D2DMoE MoE-FFN inference layer.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every
 * pointer is a DEVICE pointer unless its comment says "host".  All calls are
 * stream-ordered and asynchronous: they enqueue kernels on `stream` and return;
 * none synchronises with the host and none allocates device memory (the caller
 * owns every buffer, workspace included).
 *
 * Return value: 0 (D2D_OK) or a d2d_status code for errors detected on the host
 * before launch (bad argument, unsupported shape, launch failure).  Errors only
 * a kernel can see (a token index out of range, a bounded wait that ran out) are
 * written to the caller's device word `*dev_status` (first error wins; it stays 0
 * otherwise); the kernel then returns early instead of trapping.
 *
 * Citations name the upstream D2DMoE interface each entry point replaces, by the
 * file's path inside that project.
 *
 * Tensor layouts (row-major, innermost last), T = float (D2D_F32) or bf16 (D2D_BF16):
 *   x, out            [N, d]          T
 *   router Wa         [R, d]          T   router.layers.0.weight
 *   router Wb         [E, R]          T   router.layers.2.weight
 *   scores            [N, E]          T
 *   mask_bits         [N, ceil(E/32)] u32, bit (e%32) of word (e/32) = expert e kept
 *   offsets           [E+1]           i32, offsets[e]..offsets[e+1] = expert e's slice
 *   token_idx         [>= sum c_e]    i32, ascending token index inside each slice
 *                                     (capacity N*E covers every mask)
 *   w1 (gate), w_up   [E, d, H]       T   experts.w1   / experts.layers.{0,2}.w
 *   b1                [E, H]          T   experts.b1
 *   w2 (down)         [E, H, d]       T   experts.w2   / experts.layers.1.w
 *   last_bias         [d]             T   last_bias (shared, added once per token)
 */
#ifndef D2DMOE_H_
#define D2DMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define D2D_ABI_VERSION 2

typedef void* d2d_stream_t; /* a cudaStream_t */

enum d2d_dtype { D2D_F32 = 0, D2D_BF16 = 1 };

/* Expert activations: architectures/moe/moe_layers.py:11-16, utils.py:730-756. */
enum d2d_act { D2D_RELU = 0, D2D_GELU = 1, D2D_TANH = 2, D2D_LEAKY_RELU = 3, D2D_GELU_TANH = 4 };

enum d2d_status {
  D2D_OK = 0,
  D2D_ERR_BAD_ARG = 1,        /* null pointer, negative size, misaligned buffer */
  D2D_ERR_UNSUPPORTED = 2,    /* shape or dtype outside what the kernels cover */
  D2D_ERR_LAUNCH = 3,         /* the CUDA runtime refused a launch */
  D2D_ERR_WORKSPACE = 4,      /* workspace smaller than d2d_workspace_bytes says */
  D2D_ERR_INDEX_RANGE = 5,    /* device: a token index or offset out of range */
  D2D_ERR_TIMEOUT = 6,        /* device: a bounded wait ran out */
  D2D_ERR_NO_DEVICE = 7,      /* no sm_100 device is current */
  D2D_ERR_SCRATCH_LIMIT = 8   /* size beyond the built-in scratch of a *_noalloc entry point */
};

/* Library identity. */
int d2d_abi_version(void);
const char* d2d_strerror(int status);

/* Bytes of caller-owned workspace d2d_compact / d2d_moe_forward need for up to
 * n_max tokens.  (The upstream path allocates its scratch inside every call:
 * architectures/moe/moe_impls.py:15,190.) */
int d2d_workspace_bytes(int64_t n_max, int E, size_t* bytes /* host */);

/* Router MLP fused with the dynamic-k rule.
 * Replaces MoeficationRouter.forward (architectures/moe/moefication.py:328-330)
 * with depth 2 / ReLU / abs / no bias, followed by the 'dynk_max' branch of
 * MoeficationMoE.gate (architectures/moe/moefication.py:80-85):
 *   s = |relu(x Wa^T) Wb^T|,  keep e  iff  s_e >= T(max_e s * thresh_mult),
 * thresh_mult = (float)(1.0 - tau).  Writes mask_bits; optionally the scores
 * (scores_opt) and the initial value of the layer output
 * out_init_opt[t,:] = last_bias_opt (+ x[t,:] if add_residual), which is the
 * epilogue of MoeficationMoE.forward (architectures/moe/moefication.py:96-99)
 * moved in front of the expert scatter-add.
 * router_packed_opt: buffer made by d2d_prepack_router, or NULL. */
int d2d_router_mask(const void* x, const void* wa, const void* wb,
                    const void* router_packed_opt, float thresh_mult,
                    uint32_t* mask_bits, void* scores_opt,
                    const void* last_bias_opt, int add_residual, void* out_init_opt,
                    int64_t N, int d, int R, int E, int dtype,
                    int* dev_status, d2d_stream_t stream);

/* The dynamic-k rule alone, on given scores
 * (architectures/moe/moefication.py:80-85; the score-override hook of
 * architectures/moe/moefication.py:331-339 feeds this path). */
int d2d_mask_from_scores(const void* scores, float thresh_mult, uint32_t* mask_bits,
                         int64_t N, int E, int dtype, int* dev_status, d2d_stream_t stream);

/* The other routing rules of MoeficationMoE.gate, on given scores:
 *   D2D_RULE_TOPK  keep the k largest scores per token
 *                  (architectures/moe/moefication.py:59-63);
 *   D2D_RULE_DYNK  cumulative-share rule: shares = s / sum(s), experts in descending
 *                  share order, keep the first and every further one while the
 *                  cumulative share before it is < tau
 *                  (architectures/moe/moefication.py:64-79).
 * k is used by TOPK only (1 <= k <= E), tau by DYNK only (compared in the tensor dtype,
 * as the upstream comparison of a tensor with a Python float does). */
#define D2D_RULE_TOPK 1
#define D2D_RULE_DYNK 2
int d2d_mask_rule_from_scores(const void* scores, int rule, int k, float tau,
                              uint32_t* mask_bits, int64_t N, int E, int dtype,
                              int* dev_status, d2d_stream_t stream);

/* out[t,:] = last_bias_opt (+ x[t,:]): the epilogue of MoeficationMoE.forward
 * (architectures/moe/moefication.py:96-99) as an initial value. */
int d2d_init_out(const void* x, const void* last_bias_opt, int add_residual, void* out,
                 int64_t N, int d, int dtype, d2d_stream_t stream);

/* 0/1 routing tensor in T from the bit mask: what MoeficationMoE.forward returns
 * as gating data (architectures/moe/moefication.py:84-85,101). */
int d2d_expand_mask(const uint32_t* mask_bits, void* routing_tensor,
                    int64_t N, int E, int dtype, d2d_stream_t stream);

/* Bit mask from a 0/1 routing tensor (bit set iff routing_tensor[t,e] > 0): the
 * entry of ExpertsLayer.forward(x, routing_tensor)
 * (architectures/moe/moe_layers.py:174-177,202-204), whose caller hands over the
 * routing tensor rather than scores. */
int d2d_pack_mask(const void* routing_tensor, uint32_t* mask_bits,
                  int64_t N, int E, int dtype, d2d_stream_t stream);

/* Per-expert token lists and offsets from the bit mask.
 * Replaces CustomKernelExperts.extract_indices_atomic
 * (architectures/moe/moe_layers.py:241-249: int32 cast, argsort along tokens,
 * column sums) by a ballot / prefix-sum compaction; lists come out in ascending
 * token order.  ws: workspace of d2d_workspace_bytes(N, E). */
int d2d_compact(const uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets,
                int64_t N, int E, void* ws, size_t ws_bytes,
                int* dev_status, d2d_stream_t stream);

/* d2d_compact for callers that cannot allocate device memory and so cannot supply
 * `ws`: operator slots that receive only inputs and outputs, runtimes whose pool is
 * frozen after start-up, loops that must stay out of the driver's allocator.
 * (No counterpart upstream: the upstream path allocates its scratch inside every
 * call.)  Same outputs as d2d_compact, bit for bit.  The counts table is a fixed
 * array inside the library, held by every GPU that loads it until the process
 * exits: 1 MiB, which covers ceil(N/128) * E <= 262144 (e.g. N = 262144 with
 * E = 128); beyond that the call returns D2D_ERR_SCRATCH_LIMIT and launches
 * nothing.  It calls no allocating routine.  The first call on each device looks up
 * the array's device address (with that device current); make that first call
 * outside any stream capture.  All calls share the one array: calls that can run
 * at the same time on one GPU (different streams, no ordering) race on it. */
int d2d_compact_noalloc(const uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets,
                        int64_t N, int E, int* dev_status, d2d_stream_t stream);

/* Grouped expert FFN with fused scatter-add:
 *   for every expert e and token t in its list:
 *     out[t,:] += act(x[t,:] W1[e] + b1[e]) (* x[t,:] W_up[e]) W2[e]
 * Replaces MoeFirstLayerImplementation + MoeSecondLayerAtomicImplementation
 * (architectures/moe/moe_impls.py:8-180,183-301) as called by
 * CustomKernelExperts.forward_triton_atomic (architectures/moe/moe_layers.py:251-264);
 * with w_up_opt it covers the gated form of ExecuteAllExperts.forward
 * (architectures/moe/moe_layers.py:91-96).  The hidden activations stay on chip.
 * accumulate = 0: out is first set to last_bias_opt (+ x);  accumulate = 1: out
 * already holds its initial value (d2d_router_mask's out_init_opt) and
 * last_bias_opt / add_residual are ignored.
 * Summation order (bf16): the contributions are added to the initial value one by one in
 * the activation dtype, like upstream's atomic kernel (architectures/moe/moe_impls.py:300-301)
 * and unlike upstream's CPU path, which sums the experts first and adds last_bias and x
 * last (architectures/moe/moefication.py:96-99): a token kept by k experts sees k + 1
 * roundings at the magnitude of its output instead of one, and the order of the adds is
 * not fixed, so outputs are reproducible to that rounding, not bit for bit.  The first
 * layer rounds to T after the product, after + b1 and after the activation, as the
 * upstream CPU path does.
 * experts_packed_opt: buffer made by d2d_prepack_experts, or NULL. */
int d2d_experts_ffn(const void* x, const int32_t* token_idx, const int32_t* offsets,
                    const void* w1, const void* b1_opt, const void* w_up_opt, const void* w2,
                    const void* experts_packed_opt,
                    const void* last_bias_opt, int add_residual, int accumulate, void* out,
                    int64_t N, int d, int E, int H, int act, int dtype,
                    int* dev_status, d2d_stream_t stream);

/* d2d_experts_ffn with the labels of router training as a by-product.  Upstream runs the
 * layer in mode 'all' (every expert on every token, architectures/moe/moefication.py:56-58)
 * and captures, with forward hooks on the experts' extraction stubs / layers, the vector norm
 * over the last dimension of every expert's activations
 * (methods/dynamic_sparsification/train_routers.py:49-71,77-82; utils.py:353-369
 * torch.linalg.vector_norm(output, ord, dim=-1) -> [E, N]).  Here the expert kernel itself
 * accumulates the norm of each (expert, token) pair it computes, without materialising the
 * [E, N, d] / [E, N, H] activations:
 *   norms[e * N + t] = T(|| a_e(t) ||_ord),   a_e(t) = act(T(x[t] W1[e]) + b1[e])   (D2D_NORM_OF_INTERMEDIATE)
 *                                                   or T(h_e(t) W2[e])               (D2D_NORM_OF_OUTPUT)
 * over the T-rounded elements, fp32 accumulation, one rounding to T.  ord 1 or 2.  The call
 * first sets all E*N entries to zero; pairs outside the token lists stay zero (with the lists
 * of an all-ones routing tensor every entry is written).  Everything else as d2d_experts_ffn. */
#define D2D_NORM_OF_INTERMEDIATE 1
#define D2D_NORM_OF_OUTPUT 2
int d2d_experts_ffn_norms(const void* x, const int32_t* token_idx, const int32_t* offsets,
                          const void* w1, const void* b1_opt, const void* w_up_opt,
                          const void* w2, const void* experts_packed_opt,
                          const void* last_bias_opt, int add_residual, int accumulate, void* out,
                          void* norms, int norm_layer, int norm_ord, int64_t N, int d, int E,
                          int H, int act, int dtype, int* dev_status, d2d_stream_t stream);

/* Pre-norm fused with the block's residual: the pass in front of the layer.  An upstream
 * block runs  y = ln_2(x); y = mlp(y); return x + y  (architectures/moe/moe_models.py:69-76
 * ViT, :91-100 GPT, :148-156 Gemma).  This call reads x [N, d] once and writes
 *   xn[t,:]       = T(norm(x[t,:]))              the layer's input
 *   out_init[t,:] = T(x[t,:] + last_bias_opt)    the layer output's initial value (NULL: skip),
 * so that d2d_moe_forward(xn, ..., add_residual = D2D_OUT_PREINITIALISED, out = out_init)
 * leaves x + last_bias + sum of expert outputs in out: neither a separate residual pass nor
 * the router's initial-value writes remain.
 *   kind D2D_NORM_LAYER: (x - mean) * rsqrt(var + eps) * gamma + beta_opt (biased variance)
 *   kind D2D_NORM_RMS:   x * rsqrt(mean(x^2) + eps) * (gamma_offset + gamma); gamma_offset 1
 *                        is the Gemma form, 0 the plain one.
 * fp32 statistics, one rounding to T.  d * sizeof(T) must be a multiple of 16 and at most
 * 8192 bytes (else D2D_ERR_UNSUPPORTED); all pointers 16-byte aligned. */
#define D2D_NORM_LAYER 0
#define D2D_NORM_RMS 1
int d2d_prenorm_init(const void* x, const void* gamma, const void* beta_opt, float eps, int kind,
                     float gamma_offset, const void* last_bias_opt, void* xn, void* out_init_opt,
                     int64_t N, int d, int dtype, d2d_stream_t stream);

/* add_residual values of d2d_moe_forward: 0 = out starts as last_bias, 1 = as last_bias + x
 * (MoeficationMoE.add_residual_connection, architectures/moe/moefication.py:98-99),
 * D2D_OUT_PREINITIALISED = out already holds its initial value (d2d_prenorm_init wrote it);
 * last_bias_opt is then ignored. */
#define D2D_OUT_PREINITIALISED 2

/* The whole layer, MoeficationMoE.forward in 'dynk_max' mode
 * (architectures/moe/moefication.py:90-101): router+mask (or mask from
 * scores_in_opt when wa is NULL) -> compaction -> expert FFN.  mask_bits,
 * token_idx, offsets are outputs the caller may inspect.  routing_tensor_opt
 * [N, E] in T, or NULL: the 0/1 routing tensor the upstream forward returns as
 * gating data (architectures/moe/moefication.py:84-85,101), written by the same
 * kernel that applies the rule. */
int d2d_moe_forward(const void* x, const void* wa, const void* wb, const void* router_packed_opt,
                    const void* scores_in_opt, float thresh_mult,
                    const void* w1, const void* b1_opt, const void* w_up_opt, const void* w2,
                    const void* experts_packed_opt,
                    const void* last_bias_opt, int add_residual, void* out,
                    uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets,
                    int64_t N, int d, int R, int E, int H, int act, int dtype,
                    void* ws, size_t ws_bytes, int* dev_status,
                    void* routing_tensor_opt, d2d_stream_t stream);

/* Number of kernels the calling thread's last d2d_moe_forward issued (3 on the tensor-core
 * path: router + rule, compaction scatter, expert FFN; more on the general-shape
 * paths).  Introspection for benchmarks; no upstream counterpart. */
int d2d_last_forward_launches(void);

/* Test hook, no upstream counterpart.  Every wait inside the tensor-core kernels is bounded;
 * when one runs out the kernel writes D2D_ERR_TIMEOUT to *dev_status, frees its tensor
 * memory and returns.  wait_limit_log2 in 4..22 sets the bound to 2^n polls for later
 * launches of this process (anything else restores the default of 2^22, about a second);
 * withhold_weight_tile != 0 makes CTA 0 of later launches skip its first weight tile, so
 * that exactly this path can be exercised without faulting the GPU.  Call
 * d2d_debug_configure(0, 0) to return to normal operation. */
int d2d_debug_configure(int wait_limit_log2, int withhold_weight_tile);

/* Test hook, no upstream counterpart.  How the bf16 expert kernel brings the rows of an
 * expert's token list into shared memory: which = 0 or 1: 16-byte cp.async per row piece
 * (default, the faster one on B200); 2: TMA gathers (cp.async.bulk.tensor tile::gather4, four
 * rows per copy), kept so that the two can be compared on any workload. */
int d2d_debug_select_experts_kernel(int which);

/* One-time re-layout of the weights into the shared-memory tile images the
 * tensor-core kernels copy in bulk (bf16 only).  The upstream kernels read the
 * parameters in place (architectures/moe/moe_impls.py:137-146,276-284); here the
 * module owns a packed copy and refreshes it when the parameters change.
 * *_bytes returns 0 bytes when the shape has no tensor-core path.  `packed` must be
 * 1024-byte aligned. */
int d2d_prepack_experts_bytes(int d, int E, int H, int glu, int dtype, size_t* bytes /* host */);
int d2d_prepack_experts(const void* w1, const void* b1_opt, const void* w_up_opt, const void* w2,
                        void* packed, int d, int E, int H, int dtype, d2d_stream_t stream);
int d2d_prepack_router_bytes(int d, int R, int E, int dtype, size_t* bytes /* host */);
int d2d_prepack_router(const void* wa, const void* wb, void* packed,
                       int d, int R, int E, int dtype, d2d_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* D2DMOE_H_ */
