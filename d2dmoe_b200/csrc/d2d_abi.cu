// extern "C" entry points declared in include/d2dmoe.h: argument validation and
// dispatch to the kernels.  No device memory is allocated here and no call
// synchronises with the host.
#include "d2d_common.cuh"
#include "d2d_umma_api.cuh"

using namespace d2d;

namespace {

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline bool dtype_ok(int dt) { return dt == D2D_F32 || dt == D2D_BF16; }

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// kernels issued by the calling thread's last d2d_moe_forward
thread_local int g_last_forward_launches = 0;

}  // namespace

extern "C" {

int d2d_abi_version(void) { return D2D_ABI_VERSION; }

const char* d2d_strerror(int status) {
  switch (status) {
    case D2D_OK: return "ok";
    case D2D_ERR_BAD_ARG: return "bad argument (null pointer, negative size or misaligned buffer)";
    case D2D_ERR_UNSUPPORTED: return "shape or dtype not supported by the kernels";
    case D2D_ERR_LAUNCH: return "CUDA launch failed";
    case D2D_ERR_WORKSPACE: return "workspace too small (see d2d_workspace_bytes)";
    case D2D_ERR_INDEX_RANGE: return "device: token index or offset out of range";
    case D2D_ERR_TIMEOUT: return "device: bounded wait ran out";
    case D2D_ERR_NO_DEVICE: return "no sm_100 CUDA device is current";
    case D2D_ERR_SCRATCH_LIMIT:
      return "size exceeds the built-in scratch array of the no-allocation entry point "
             "(ceil(N/128)*E must be <= 262144); use d2d_compact with a caller workspace";
    default: return "unknown status";
  }
}

int d2d_workspace_bytes(int64_t n_max, int E, size_t* bytes) {
  if (!bytes || n_max < 0 || E < 1) return D2D_ERR_BAD_ARG;
  *bytes = align_up(compact_workspace_bytes(n_max, E), 256);
  return D2D_OK;
}

int d2d_router_mask(const void* x, const void* wa, const void* wb, const void* router_packed_opt,
                    float thresh_mult, uint32_t* mask_bits, void* scores_opt,
                    const void* last_bias_opt, int add_residual, void* out_init_opt, int64_t N,
                    int d, int R, int E, int dtype, int* dev_status, d2d_stream_t stream) {
  if (!x || !wa || !wb || !mask_bits || N < 0 || d < 1 || R < 1 || E < 1) return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (N == 0) return D2D_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // the tensor-core router moves x, last_bias and the output's initial value in 16-byte
  // pieces; buffers that do not allow that take the general-shape kernel
  if (router_packed_opt && umma_router_supported(d, R, E, dtype) && aligned(x, 16) &&
      aligned(last_bias_opt, 16) && aligned(out_init_opt, 16) && aligned(router_packed_opt, 1024))
    return launch_router_mask_umma(x, router_packed_opt, thresh_mult, mask_bits, scores_opt,
                                   nullptr, last_bias_opt, add_residual, out_init_opt, nullptr, N, d, R, E,
                                   dev_status, s);
  return launch_router_mask_simt(x, wa, wb, thresh_mult, mask_bits, scores_opt, last_bias_opt,
                                 add_residual, out_init_opt, N, d, R, E, dtype, dev_status, s);
}

int d2d_mask_from_scores(const void* scores, float thresh_mult, uint32_t* mask_bits, int64_t N,
                         int E, int dtype, int* dev_status, d2d_stream_t stream) {
  if (!scores || !mask_bits || N < 0 || E < 1) return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (N == 0) return D2D_OK;
  return launch_mask_from_scores(scores, thresh_mult, mask_bits, N, E, dtype, dev_status,
                                 (cudaStream_t)stream);
}

int d2d_mask_rule_from_scores(const void* scores, int rule, int k, float tau, uint32_t* mask_bits,
                              int64_t N, int E, int dtype, int* dev_status, d2d_stream_t stream) {
  if (!scores || !mask_bits || N < 0 || E < 1) return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (rule == D2D_RULE_TOPK) {
    if (k < 1 || k > E) return D2D_ERR_BAD_ARG;      // torch.topk raises for k out of range
  } else if (rule != D2D_RULE_DYNK) {
    return D2D_ERR_BAD_ARG;
  }
  (void)dev_status;
  if (N == 0) return D2D_OK;
  return launch_gate_rule(scores, rule, k, tau, mask_bits, N, E, dtype, (cudaStream_t)stream);
}

int d2d_init_out(const void* x, const void* last_bias_opt, int add_residual, void* out, int64_t N,
                 int d, int dtype, d2d_stream_t stream) {
  if (!out || N < 0 || d < 1 || (add_residual && !x)) return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (N == 0) return D2D_OK;
  return launch_init_out(x, last_bias_opt, add_residual, out, N, d, dtype, (cudaStream_t)stream);
}

int d2d_prenorm_init(const void* x, const void* gamma, const void* beta_opt, float eps, int kind,
                     float gamma_offset, const void* last_bias_opt, void* xn, void* out_init_opt,
                     int64_t N, int d, int dtype, d2d_stream_t stream) {
  if (!x || !gamma || !xn || N < 0 || d < 1 || (kind != D2D_NORM_LAYER && kind != D2D_NORM_RMS))
    return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (N == 0) return D2D_OK;
  return launch_prenorm_init(x, gamma, beta_opt, eps, kind, gamma_offset, last_bias_opt, xn,
                             out_init_opt, N, d, dtype, (cudaStream_t)stream);
}

int d2d_expand_mask(const uint32_t* mask_bits, void* routing_tensor, int64_t N, int E, int dtype,
                    d2d_stream_t stream) {
  if (!mask_bits || !routing_tensor || N < 0 || E < 1) return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (N == 0) return D2D_OK;
  return launch_expand_mask(mask_bits, routing_tensor, N, E, dtype, (cudaStream_t)stream);
}

int d2d_pack_mask(const void* routing_tensor, uint32_t* mask_bits, int64_t N, int E, int dtype,
                  d2d_stream_t stream) {
  if (!mask_bits || !routing_tensor || N < 0 || E < 1) return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return D2D_ERR_UNSUPPORTED;
  if (N == 0) return D2D_OK;
  return launch_pack_mask(routing_tensor, mask_bits, N, E, dtype, (cudaStream_t)stream);
}

int d2d_compact(const uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets, int64_t N, int E,
                void* ws, size_t ws_bytes, int* dev_status, d2d_stream_t stream) {
  if (!mask_bits || !token_idx || !offsets || !ws || N < 0 || E < 1) return D2D_ERR_BAD_ARG;
  if (!aligned(ws, 16)) return D2D_ERR_BAD_ARG;
  if (ws_bytes < compact_workspace_bytes(N, E)) return D2D_ERR_WORKSPACE;
  return launch_compact(mask_bits, token_idx, offsets, N, E, (int32_t*)ws, dev_status,
                        (cudaStream_t)stream, false);
}

static int experts_ffn_impl(const void* x, const int32_t* token_idx, const int32_t* offsets,
                            const void* w1, const void* b1_opt, const void* w_up_opt,
                            const void* w2, const void* experts_packed_opt,
                            const void* last_bias_opt, int add_residual, int accumulate,
                            void* out, NormCapture nc, int64_t N, int d, int E, int H, int act,
                            int dtype, int* dev_status, d2d_stream_t stream) {
  if (!x || !token_idx || !offsets || !w1 || !w2 || !out || N < 0 || d < 1 || E < 1 || H < 1)
    return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype) || act < D2D_RELU || act > D2D_GELU_TANH) return D2D_ERR_UNSUPPORTED;
  if (!aligned(out, 16) || !aligned(x, 16)) return D2D_ERR_BAD_ARG;
  if (nc.layer != 0 &&
      (!nc.norms || !aligned(nc.norms, 4) || (nc.ord != 1 && nc.ord != 2) ||
       (nc.layer != D2D_NORM_OF_INTERMEDIATE && nc.layer != D2D_NORM_OF_OUTPUT)))
    return D2D_ERR_BAD_ARG;
  if (N == 0) return D2D_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (nc.layer != 0 &&
      cudaMemsetAsync(nc.norms, 0, (size_t)N * E * (dtype == D2D_F32 ? 4 : 2), s) != cudaSuccess)
    return D2D_ERR_LAUNCH;
  if (!accumulate) {
    int rc = launch_init_out(x, last_bias_opt, add_residual, out, N, d, dtype, s);
    if (rc != D2D_OK) return rc;
  }
  if (experts_packed_opt && umma_experts_supported(d, E, H, w_up_opt != nullptr, dtype) &&
      aligned(experts_packed_opt, 1024))
    return launch_experts_umma(x, token_idx, offsets, experts_packed_opt, out, N, d, E, H,
                               w_up_opt != nullptr, act, dev_status, s, nc);
  return launch_experts_simt(x, token_idx, offsets, w1, b1_opt, w_up_opt, w2, out, N, d, E, H, act,
                             dtype, dev_status, s, nc);
}

int d2d_experts_ffn(const void* x, const int32_t* token_idx, const int32_t* offsets,
                    const void* w1, const void* b1_opt, const void* w_up_opt, const void* w2,
                    const void* experts_packed_opt, const void* last_bias_opt, int add_residual,
                    int accumulate, void* out, int64_t N, int d, int E, int H, int act, int dtype,
                    int* dev_status, d2d_stream_t stream) {
  return experts_ffn_impl(x, token_idx, offsets, w1, b1_opt, w_up_opt, w2, experts_packed_opt,
                          last_bias_opt, add_residual, accumulate, out, NormCapture(), N, d, E, H,
                          act, dtype, dev_status, stream);
}

int d2d_experts_ffn_norms(const void* x, const int32_t* token_idx, const int32_t* offsets,
                          const void* w1, const void* b1_opt, const void* w_up_opt,
                          const void* w2, const void* experts_packed_opt,
                          const void* last_bias_opt, int add_residual, int accumulate, void* out,
                          void* norms, int norm_layer, int norm_ord, int64_t N, int d, int E,
                          int H, int act, int dtype, int* dev_status, d2d_stream_t stream) {
  NormCapture nc;
  nc.norms = norms;
  nc.layer = norm_layer;
  nc.ord = norm_ord;
  if (norm_layer == 0) return D2D_ERR_BAD_ARG;
  return experts_ffn_impl(x, token_idx, offsets, w1, b1_opt, w_up_opt, w2, experts_packed_opt,
                          last_bias_opt, add_residual, accumulate, out, nc, N, d, E, H, act, dtype,
                          dev_status, stream);
}

int d2d_moe_forward(const void* x, const void* wa, const void* wb, const void* router_packed_opt,
                    const void* scores_in_opt, float thresh_mult, const void* w1,
                    const void* b1_opt, const void* w_up_opt, const void* w2,
                    const void* experts_packed_opt, const void* last_bias_opt, int add_residual,
                    void* out, uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets,
                    int64_t N, int d, int R, int E, int H, int act, int dtype, void* ws,
                    size_t ws_bytes, int* dev_status, void* routing_tensor_opt,
                    d2d_stream_t stream) {
  int rc, nl = 0;
  bool counts_ready = false, rt_done = routing_tensor_opt == nullptr;
  g_last_forward_launches = 0;
  if (!wa && !scores_in_opt) return D2D_ERR_BAD_ARG;
  if (!mask_bits || !token_idx || !offsets || !ws || !aligned(ws, 16)) return D2D_ERR_BAD_ARG;
  // every argument check of the later stages comes before the first launch
  if (!x || !w1 || !w2 || !out || N < 0 || d < 1 || E < 1 || H < 1) return D2D_ERR_BAD_ARG;
  if (!aligned(out, 16) || !aligned(x, 16) || !aligned(mask_bits, 4) || !aligned(token_idx, 4) ||
      !aligned(offsets, 4))
    return D2D_ERR_BAD_ARG;
  if (!dtype_ok(dtype) || act < D2D_RELU || act > D2D_GELU_TANH) return D2D_ERR_UNSUPPORTED;
  if (ws_bytes < compact_workspace_bytes(N, E)) return D2D_ERR_WORKSPACE;
  if (add_residual < 0 || add_residual > D2D_OUT_PREINITIALISED) return D2D_ERR_BAD_ARG;
  if (N == 0) return D2D_OK;
  // out already initialised by the caller (d2d_prenorm_init): the first kernel writes no rows
  const bool pre = add_residual == D2D_OUT_PREINITIALISED;
  void* out_init = pre ? nullptr : out;
  if (pre) {
    add_residual = 0;
    last_bias_opt = nullptr;
  }
  if (scores_in_opt) {
    // rule + counts table + output init in one launch when the shape allows it
    rc = launch_gate_scores_fused(scores_in_opt, thresh_mult, mask_bits, routing_tensor_opt,
                                  (int32_t*)ws, x, last_bias_opt, add_residual, out_init, N, d, E,
                                  dtype, (cudaStream_t)stream);
    if (rc == D2D_OK) {
      counts_ready = true;
      rt_done = true;
      nl += 1;
    } else if (rc == D2D_ERR_UNSUPPORTED) {
      rc = d2d_mask_from_scores(scores_in_opt, thresh_mult, mask_bits, N, E, dtype, dev_status,
                                stream);
      if (rc != D2D_OK) return rc;
      nl += 1;
      if (!pre) {
        rc = d2d_init_out(x, last_bias_opt, add_residual, out, N, d, dtype, stream);
        nl += 1;
      }
    }
  } else if (router_packed_opt && wb && R >= 1 && umma_router_supported(d, R, E, dtype) &&
             aligned(last_bias_opt, 16) && aligned(router_packed_opt, 1024)) {
    // the tensor-core router also fills the compaction's counts table
    rc = launch_router_mask_umma(x, router_packed_opt, thresh_mult, mask_bits, nullptr,
                                 routing_tensor_opt, last_bias_opt, add_residual, out_init,
                                 (int32_t*)ws, N, d, R, E, dev_status, (cudaStream_t)stream);
    counts_ready = true;
    rt_done = true;
    nl += 1;
  } else {
    // general-shape router: mask bits, routing tensor and the output's initial value
    if (!wb || R < 1) return D2D_ERR_BAD_ARG;
    rc = launch_router_mask_simt(x, wa, wb, thresh_mult, mask_bits, nullptr, last_bias_opt,
                                 add_residual, out_init, N, d, R, E, dtype, dev_status,
                                 (cudaStream_t)stream, routing_tensor_opt);
    rt_done = true;
    nl += 1;
  }
  if (rc != D2D_OK) return rc;
  rc = launch_compact(mask_bits, token_idx, offsets, N, E, (int32_t*)ws, dev_status,
                      (cudaStream_t)stream, counts_ready);
  if (rc != D2D_OK) return rc;
  nl += counts_ready ? 1 : 2;      // [count,] scatter
  if (!rt_done) {                  // paths whose first kernel does not write the routing tensor
    rc = launch_expand_mask(mask_bits, routing_tensor_opt, N, E, dtype, (cudaStream_t)stream);
    if (rc != D2D_OK) return rc;
    nl += 1;
  }
  g_last_forward_launches = nl + 1;
  return d2d_experts_ffn(x, token_idx, offsets, w1, b1_opt, w_up_opt, w2, experts_packed_opt,
                         nullptr, 0, /*accumulate=*/1, out, N, d, E, H, act, dtype, dev_status,
                         stream);
}

int d2d_last_forward_launches(void) { return g_last_forward_launches; }

int d2d_debug_select_experts_kernel(int which) {
  umma_debug_select_experts_kernel(which);
  return D2D_OK;
}

int d2d_debug_configure(int wait_limit_log2, int withhold_weight_tile) {
  umma_debug_configure(wait_limit_log2, withhold_weight_tile);
  return D2D_OK;
}

int d2d_prepack_experts_bytes(int d, int E, int H, int glu, int dtype, size_t* bytes) {
  if (!bytes || d < 1 || E < 1 || H < 1) return D2D_ERR_BAD_ARG;
  *bytes = umma_experts_supported(d, E, H, glu != 0, dtype) ? umma_experts_packed_bytes(d, E, H, glu != 0) : 0;
  return D2D_OK;
}

int d2d_prepack_experts(const void* w1, const void* b1_opt, const void* w_up_opt, const void* w2,
                        void* packed, int d, int E, int H, int dtype, d2d_stream_t stream) {
  if (!w1 || !w2 || !packed) return D2D_ERR_BAD_ARG;
  if (!umma_experts_supported(d, E, H, w_up_opt != nullptr, dtype)) return D2D_ERR_UNSUPPORTED;
  if (!aligned(packed, 1024)) return D2D_ERR_BAD_ARG;
  return launch_prepack_experts(w1, b1_opt, w_up_opt, w2, packed, d, E, H, (cudaStream_t)stream);
}

int d2d_prepack_router_bytes(int d, int R, int E, int dtype, size_t* bytes) {
  if (!bytes || d < 1 || R < 1 || E < 1) return D2D_ERR_BAD_ARG;
  *bytes = umma_router_supported(d, R, E, dtype) ? umma_router_packed_bytes(d, R, E) : 0;
  return D2D_OK;
}

int d2d_prepack_router(const void* wa, const void* wb, void* packed, int d, int R, int E,
                       int dtype, d2d_stream_t stream) {
  if (!wa || !wb || !packed) return D2D_ERR_BAD_ARG;
  if (!umma_router_supported(d, R, E, dtype)) return D2D_ERR_UNSUPPORTED;
  if (!aligned(packed, 1024)) return D2D_ERR_BAD_ARG;
  return launch_prepack_router(wa, wb, packed, d, R, E, (cudaStream_t)stream);
}

}  // extern "C"
