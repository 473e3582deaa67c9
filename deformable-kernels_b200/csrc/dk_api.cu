// extern "C" surface of the library (see include/dk_b200.h): argument checks, dtype
// dispatch, workspace carving.  No allocation, no synchronisation, no printing.
#include <mutex>

#include "dk_common.cuh"

namespace dk {

static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return DK_ERR_CUDA;
  }
  return DK_OK;
}

namespace {
struct DevAttr {
  bool known = false;
  // without a device (host-only plan queries) the figures of the one target, B200: 227 KB opt-in, 148 SMs
  int smem_optin = 227 * 1024;
  int sms = 148;
};
std::mutex g_attr_mutex;
DevAttr g_attr[64];

const DevAttr& attrs() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> lock(g_attr_mutex);
  DevAttr& a = g_attr[dev];
  if (!a.known) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess && v > 0) a.smem_optin = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) a.sms = v;
    a.known = true;
  }
  return a;
}
}  // namespace

int device_smem_optin() { return attrs().smem_optin; }
int device_sm_count() { return attrs().sms; }

bool make_geom(const dk_geom* in, Geom* g) {
  if (!in) return false;
  if (in->batch <= 0 || in->channels <= 0 || in->in_h <= 0 || in->in_w <= 0) return false;
  if (in->kernel_h <= 0 || in->kernel_w <= 0 || in->stride_h <= 0 || in->stride_w <= 0) return false;
  if (in->pad_h < 0 || in->pad_w < 0 || in->dil_h <= 0 || in->dil_w <= 0) return false;
  if (in->scope_h <= 0 || in->scope_w <= 0 || in->rotation_groups <= 0) return false;
  if (in->channels % in->rotation_groups != 0) return false;
  g->N = in->batch; g->C = in->channels; g->H = in->in_h; g->W = in->in_w;
  g->kH = in->kernel_h; g->kW = in->kernel_w; g->sH = in->stride_h; g->sW = in->stride_w;
  g->pH = in->pad_h; g->pW = in->pad_w; g->dH = in->dil_h; g->dW = in->dil_w;
  g->scH = in->scope_h; g->scW = in->scope_w; g->G = in->rotation_groups;
  const long long eh = (long long)g->H + 2LL * g->pH - ((long long)g->dH * (g->kH - 1) + 1);
  const long long ew = (long long)g->W + 2LL * g->pW - ((long long)g->dW * (g->kW - 1) + 1);
  if (eh < 0 || ew < 0) return false;  // "convolution input is too small"
  g->Ho = (int)(eh / g->sH) + 1;
  g->Wo = (int)(ew / g->sW) + 1;
  const long long taps = (long long)g->kH * g->kW, P = (long long)g->Ho * g->Wo, HW = (long long)g->H * g->W;
  const long long cells = (long long)g->scH * g->scW;
  if (taps > 4096 || P > 0x3fffffffLL || HW > 0x3fffffffLL || cells > 65536) return false;
  // per-sample offset planes are indexed with 32-bit arithmetic inside a sample
  if (taps * 2 * P * g->G > 0x7fffffffLL) return false;
  g->taps = (int)taps; g->P = (int)P; g->HW = (int)HW; g->cells = (int)cells;
  g->Cg = g->C / g->G;
  return true;
}

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
static inline size_t acc_bytes(int dtype) { return dtype == DK_F64 ? 8 : 4; }
static inline bool dtype_ok(int dtype) { return dtype == DK_F32 || dtype == DK_F16 || dtype == DK_F64; }

}  // namespace dk

using namespace dk;

#define DK_DISPATCH(dtype, EXPR)                         \
  switch (dtype) {                                       \
    case DK_F32: { using T = float; return (EXPR); }     \
    case DK_F16: { using T = __half; return (EXPR); }    \
    case DK_F64: { using T = double; return (EXPR); }    \
    default: return DK_ERR_BAD_ARGUMENT;                 \
  }
#define P_(T, p) reinterpret_cast<const T*>(p)
#define M_(T, p) reinterpret_cast<T*>(p)

extern "C" {

const char* dk_status_string(int status) {
  switch (status) {
    case DK_OK: return "ok";
    case DK_ERR_BAD_ARGUMENT: return "bad argument";
    case DK_ERR_UNSUPPORTED: return "unsupported shape or size";
    case DK_ERR_WORKSPACE: return "workspace missing or too small";
    case DK_ERR_CUDA: return "CUDA error";
    default: return "unknown status";
  }
}

int dk_last_cuda_error(void) { return g_last_cuda_error; }
const char* dk_version(void) { return "dk_b200 0.1 (sm_100a)"; }

int dk_local_plan_query(const dk_geom* g, int dtype, int pass, long long* out8) {
  Geom gg;
  if (!out8 || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  if (dtype != DK_F16 || !mma_path_enabled()) return DK_ERR_UNSUPPORTED;
  if (pass >= 4 && pass <= 7) return local_ring_plan_query(gg, pass, out8);
  return local_mma_plan_query(gg, pass, out8);
}

int dk_ring_error_status(void) { return ring_error_status(); }

int dk_output_size(const dk_geom* g, int* out_h, int* out_w) {
  Geom gg;
  if (!make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  if (out_h) *out_h = gg.Ho;
  if (out_w) *out_w = gg.Wo;
  return DK_OK;
}

/* ---------------------------------------------------------------- local DK */

int dk_sample_depthwise_forward(const void* input, const void* rotation, const void* filter, void* output,
                                const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!input || !rotation || !filter || !output || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, local_forward<T>(P_(T, input), P_(T, rotation), P_(T, filter), M_(T, output), gg, (cudaStream_t)stream))
}

int dk_sample_depthwise_backward_data(const void* grad_output, const void* rotation, const void* filter,
                                      void* grad_input, const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!grad_output || !rotation || !filter || !grad_input || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, local_backward_data<T>(P_(T, grad_output), P_(T, rotation), P_(T, filter), M_(T, grad_input), gg,
                                            (cudaStream_t)stream))
}

size_t dk_sample_depthwise_backward_filter_workspace_bytes(const dk_geom* g, int dtype) {
  Geom gg;
  if (!make_geom(g, &gg) || !dtype_ok(dtype)) return 0;
  size_t need = filter_plan(gg, acc_bytes(dtype)).ws_bytes;
  if (dtype == DK_F16) {
    const size_t fast = local_filter_mma_workspace(gg);
    if (fast > need) need = fast;
  }
  return align256(need);
}

int dk_sample_depthwise_backward_filter(const void* grad_output, const void* input, const void* rotation,
                                        void* grad_filter, const dk_geom* g, int dtype, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  Geom gg;
  if (!grad_output || !input || !rotation || !grad_filter || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, local_backward_filter<T>(P_(T, grad_output), P_(T, input), P_(T, rotation), M_(T, grad_filter), gg,
                                              workspace, workspace_bytes, (cudaStream_t)stream))
}

size_t dk_sample_depthwise_backward_rotation_workspace_bytes(const dk_geom* g, int dtype) {
  Geom gg;
  if (!make_geom(g, &gg) || !dtype_ok(dtype)) return 0;
  return dtype == DK_F16 ? align256(local_rot_mma_workspace(gg)) : 0;
}

int dk_sample_depthwise_backward_rotation(const void* grad_output, const void* input, const void* rotation,
                                          const void* filter, void* grad_rotation, const dk_geom* g, int dtype,
                                          void* workspace, size_t workspace_bytes, void* stream) {
  Geom gg;
  if (!grad_output || !input || !rotation || !filter || !grad_rotation || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, local_backward_rotation<T>(P_(T, grad_output), P_(T, input), P_(T, rotation), P_(T, filter),
                                                M_(T, grad_rotation), gg, workspace, workspace_bytes, (cudaStream_t)stream))
}

size_t dk_sample_depthwise_backward_workspace_bytes(const dk_geom* g, int dtype) {
  const size_t a = dk_sample_depthwise_backward_filter_workspace_bytes(g, dtype);
  const size_t b = dk_sample_depthwise_backward_rotation_workspace_bytes(g, dtype);
  size_t need = a > b ? a : b;  // the passes run one after the other on the stream and share the buffer
  Geom gg;
  if (dtype == DK_F16 && make_geom(g, &gg)) {
    const size_t c = align256(local_gw_ring_workspace(gg)), d = align256(local_bwd_ring_workspace(gg));
    const size_t e = align256(local_gw_mma_workspace(gg));
    if (c > need) need = c;
    if (d > need) need = d;
    if (e > need) need = e;
  }
  return need;
}

int dk_sample_depthwise_backward(const void* grad_output, const void* input, const void* rotation, const void* filter,
                                 void* grad_input, void* grad_rotation, void* grad_filter, const dk_geom* g, int dtype,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (!dtype_ok(dtype)) return DK_ERR_BAD_ARGUMENT;
  int rc = DK_OK;
  if (grad_input && grad_rotation && grad_filter && dtype == DK_F16 && mma_path_enabled()) {
    // the whole backward in one pass over grad_output, input and the offsets, where that is the faster way
    Geom gg;
    if (!grad_output || !input || !rotation || !filter || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
    if (local_bwd_ring_preferred(gg)) {
      rc = local_bwd_ring(P_(__half, grad_output), P_(__half, input), P_(__half, rotation), P_(__half, filter),
                          M_(__half, grad_input), M_(__half, grad_rotation), M_(__half, grad_filter), gg, workspace,
                          workspace_bytes, (cudaStream_t)stream);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  if (grad_input) {
    rc = dk_sample_depthwise_backward_data(grad_output, rotation, filter, grad_input, g, dtype, stream);
    if (rc) return rc;
  }
  if (grad_rotation && grad_filter && dtype == DK_F16 && mma_path_enabled()) {
    // both remaining gradients consume the products dy * x: one pass over dy, x and the offsets where the shape allows
    Geom gg;
    if (!grad_output || !input || !rotation || !filter || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
    rc = local_gw_ring(P_(__half, grad_output), P_(__half, input), P_(__half, rotation), P_(__half, filter),
                       M_(__half, grad_rotation), M_(__half, grad_filter), gg, workspace, workspace_bytes, (cudaStream_t)stream);
    if (rc != DK_ERR_UNSUPPORTED) return rc;
    rc = local_gw_mma(P_(__half, grad_output), P_(__half, input), P_(__half, rotation), P_(__half, filter),
                      M_(__half, grad_rotation), M_(__half, grad_filter), gg, workspace, workspace_bytes, (cudaStream_t)stream);
    if (rc != DK_ERR_UNSUPPORTED) return rc;
  }
  if (grad_rotation) {
    rc = dk_sample_depthwise_backward_rotation(grad_output, input, rotation, filter, grad_rotation, g, dtype, workspace,
                                               workspace_bytes, stream);
    if (rc) return rc;
  }
  if (grad_filter) {
    rc = dk_sample_depthwise_backward_filter(grad_output, input, rotation, grad_filter, g, dtype, workspace,
                                             workspace_bytes, stream);
  }
  return rc;
}

int dk_sample_depthwise_backward_one_pass(const void* grad_output, const void* input, const void* rotation, const void* filter,
                                          void* grad_input, void* grad_rotation, void* grad_filter, const dk_geom* g, int dtype,
                                          void* workspace, size_t workspace_bytes, void* stream) {
  Geom gg;
  if (!grad_output || !input || !rotation || !filter || !grad_input || !grad_rotation || !grad_filter || !make_geom(g, &gg))
    return DK_ERR_BAD_ARGUMENT;
  if (dtype != DK_F16 || !mma_path_enabled()) return DK_ERR_UNSUPPORTED;
  return local_bwd_ring(P_(__half, grad_output), P_(__half, input), P_(__half, rotation), P_(__half, filter),
                        M_(__half, grad_input), M_(__half, grad_rotation), M_(__half, grad_filter), gg, workspace, workspace_bytes,
                        (cudaStream_t)stream);
}

/* ---------------------------------------------------------------- DK + DCN */

int dk_deform_sample_depthwise_forward(const void* input, const void* offset, const void* rotation, const void* filter,
                                       void* output, const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!input || !offset || !filter || !output || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  if (!rotation) {  // zero kernel-space offsets: tensor-core path only, the caller falls back to a tensor of zeros
    if (dtype != DK_F16 || !mma_path_enabled()) return DK_ERR_UNSUPPORTED;
    return deform_forward_mma(P_(__half, input), P_(__half, offset), nullptr, P_(__half, filter), M_(__half, output), gg,
                              (cudaStream_t)stream);
  }
  DK_DISPATCH(dtype, deform_forward<T>(P_(T, input), P_(T, offset), P_(T, rotation), P_(T, filter), M_(T, output), gg,
                                       (cudaStream_t)stream))
}

size_t dk_deform_sample_depthwise_backward_data_workspace_bytes(const dk_geom* g, int dtype) {
  Geom gg;
  if (!make_geom(g, &gg) || !dtype_ok(dtype)) return 0;
  if (dtype != DK_F16) return 0;
  return align256((size_t)gg.N * gg.C * gg.HW * sizeof(float));
}

int dk_deform_sample_depthwise_backward_data(const void* grad_output, const void* offset, const void* rotation,
                                             const void* filter, void* grad_input, const dk_geom* g, int dtype,
                                             void* workspace, size_t workspace_bytes, void* stream) {
  Geom gg;
  if (!grad_output || !offset || !rotation || !filter || !grad_input || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, deform_backward_data<T>(P_(T, grad_output), P_(T, offset), P_(T, rotation), P_(T, filter),
                                             M_(T, grad_input), gg, workspace, workspace_bytes, (cudaStream_t)stream))
}

size_t dk_deform_sample_depthwise_backward_filter_workspace_bytes(const dk_geom* g, int dtype) {
  Geom gg;
  if (!make_geom(g, &gg) || !dtype_ok(dtype)) return 0;
  size_t need = filter_plan(gg, acc_bytes(dtype)).ws_bytes;
  const size_t plane = deform_filter_plane_workspace(gg, dtype);
  if (plane > need) need = plane;
  if (dtype == DK_F16) {
    const size_t fast = deform_filter_mma_workspace(gg);
    if (fast > need) need = fast;
    const size_t fused = deform_coords_bank_workspace(gg);  // the bank gradient riding along with the offset gradients
    if (fused > need) need = fused;
  }
  return align256(need);
}

int dk_deform_sample_depthwise_backward_filter(const void* grad_output, const void* input, const void* offset,
                                               const void* rotation, void* grad_filter, const dk_geom* g, int dtype,
                                               void* workspace, size_t workspace_bytes, void* stream) {
  Geom gg;
  if (!grad_output || !input || !offset || !rotation || !grad_filter || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, deform_backward_filter<T>(P_(T, grad_output), P_(T, input), P_(T, offset), P_(T, rotation),
                                               M_(T, grad_filter), gg, workspace, workspace_bytes, (cudaStream_t)stream))
}

int dk_deform_sample_depthwise_backward_offset(const void* grad_output, const void* input, const void* offset,
                                               const void* rotation, const void* filter, void* grad_offset,
                                               const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!grad_output || !input || !offset || !rotation || !filter || !grad_offset || !make_geom(g, &gg))
    return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, deform_backward_coords<T>(P_(T, grad_output), P_(T, input), P_(T, offset), P_(T, rotation),
                                               P_(T, filter), M_(T, grad_offset), (T*)nullptr, gg, (cudaStream_t)stream))
}

int dk_deform_sample_depthwise_backward_rotation(const void* grad_output, const void* input, const void* offset,
                                                 const void* rotation, const void* filter, void* grad_rotation,
                                                 const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!grad_output || !input || !offset || !rotation || !filter || !grad_rotation || !make_geom(g, &gg))
    return DK_ERR_BAD_ARGUMENT;
  DK_DISPATCH(dtype, deform_backward_coords<T>(P_(T, grad_output), P_(T, input), P_(T, offset), P_(T, rotation),
                                               P_(T, filter), (T*)nullptr, M_(T, grad_rotation), gg, (cudaStream_t)stream))
}

/* First region of the fused backward's workspace: used by grad-input, then (same stream) by the offset gradients. */
static size_t deform_front_ws(const dk_geom* g, int dtype) {
  size_t need = dk_deform_sample_depthwise_backward_data_workspace_bytes(g, dtype);
  Geom gg;
  if (dtype == DK_F16 && make_geom(g, &gg)) {
    const size_t c = align256(deform_coords_mma_workspace(gg));
    if (c > need) need = c;
  }
  return need;
}

size_t dk_deform_sample_depthwise_backward_workspace_bytes(const dk_geom* g, int dtype) {
  return deform_front_ws(g, dtype) + dk_deform_sample_depthwise_backward_filter_workspace_bytes(g, dtype);
}

static int deform_coords_dispatch(const void* grad_output, const void* input, const void* offset, const void* rotation,
                                  const void* filter, void* grad_offset, void* grad_rotation, const Geom& gg, int dtype,
                                  void* stream) {
  DK_DISPATCH(dtype, deform_backward_coords<T>(P_(T, grad_output), P_(T, input), P_(T, offset), P_(T, rotation),
                                               P_(T, filter), M_(T, grad_offset), M_(T, grad_rotation), gg,
                                               (cudaStream_t)stream))
}

int dk_deform_sample_depthwise_backward(const void* grad_output, const void* input, const void* offset,
                                        const void* rotation, const void* filter, void* grad_input, void* grad_offset,
                                        void* grad_rotation, void* grad_filter, const dk_geom* g, int dtype,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  Geom gg;
  if (!grad_output || !input || !offset || !filter || !make_geom(g, &gg) || !dtype_ok(dtype)) return DK_ERR_BAD_ARGUMENT;
  const size_t data_ws = deform_front_ws(g, dtype);
  const size_t filt_ws = dk_deform_sample_depthwise_backward_filter_workspace_bytes(g, dtype);
  int rc = DK_OK;
  if (!rotation) {  // zero kernel-space offsets (see the forward); nothing to differentiate with respect to them
    if (grad_rotation) return DK_ERR_BAD_ARGUMENT;
    if (dtype != DK_F16 || !mma_path_enabled()) return DK_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < data_ws + filt_ws) return DK_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    if (grad_input) {
      rc = deform_data_mma(P_(__half, grad_output), P_(__half, offset), nullptr, P_(__half, filter), M_(__half, grad_input),
                           gg, workspace, data_ws, s);
      if (rc) return rc;
    }
    bool bank_done = false;
    if (grad_offset) {
      rc = deform_coords_mma(P_(__half, grad_output), P_(__half, input), P_(__half, offset), nullptr, P_(__half, filter),
                             M_(__half, grad_offset), nullptr, gg, workspace, data_ws, s, M_(__half, grad_filter),
                             (char*)workspace + data_ws, filt_ws, &bank_done);
      if (rc) return rc;
    }
    if (grad_filter && !bank_done)
      rc = deform_filter_mma(P_(__half, grad_output), P_(__half, input), P_(__half, offset), nullptr, M_(__half, grad_filter),
                             gg, (char*)workspace + data_ws, filt_ws, s);
    return rc;
  }
  if (grad_input) {
    if (data_ws && (!workspace || workspace_bytes < data_ws)) return DK_ERR_WORKSPACE;
    rc = dk_deform_sample_depthwise_backward_data(grad_output, offset, rotation, filter, grad_input, g, dtype, workspace,
                                                  data_ws, stream);
    if (rc) return rc;
  }
  bool bank_done = false;
  if (grad_offset || grad_rotation) {
    rc = DK_ERR_UNSUPPORTED;
    if (dtype == DK_F16 && mma_path_enabled() && workspace && workspace_bytes >= data_ws) {
      const bool room = grad_filter && workspace_bytes >= data_ws + filt_ws;
      rc = deform_coords_mma(P_(__half, grad_output), P_(__half, input), P_(__half, offset), P_(__half, rotation),
                             P_(__half, filter), M_(__half, grad_offset), M_(__half, grad_rotation), gg, workspace, data_ws,
                             (cudaStream_t)stream, room ? M_(__half, grad_filter) : nullptr, (char*)workspace + data_ws,
                             room ? filt_ws : 0, &bank_done);
    }
    if (rc == DK_ERR_UNSUPPORTED)
      rc = deform_coords_dispatch(grad_output, input, offset, rotation, filter, grad_offset, grad_rotation, gg, dtype, stream);
    if (rc) return rc;
  }
  if (grad_filter && !bank_done) {
    if (!workspace || workspace_bytes < data_ws + filt_ws) return DK_ERR_WORKSPACE;
    rc = dk_deform_sample_depthwise_backward_filter(grad_output, input, offset, rotation, grad_filter, g, dtype,
                                                    (char*)workspace + data_ws, filt_ws, stream);
  }
  return rc;
}

/* ---------------------------------------------------------------- N-d linear sample */

static int nd_args(int batch, int channels, int dims, const int* shape, NdShape* sh, int* prod) {
  if (batch <= 0 || channels <= 0 || dims <= 0 || !shape) return DK_ERR_BAD_ARGUMENT;
  if (dims > kMaxNdDims) return DK_ERR_UNSUPPORTED;
  long long p = 1;
  for (int d = 0; d < kMaxNdDims; ++d) sh->s[d] = 1;
  for (int d = 0; d < dims; ++d) {
    if (shape[d] <= 0) return DK_ERR_BAD_ARGUMENT;
    sh->s[d] = shape[d];
    p *= shape[d];
    if (p > 0x3fffffffLL) return DK_ERR_UNSUPPORTED;
  }
  *prod = (int)p;
  return DK_OK;
}

int dk_nd_linear_sample_forward(const void* data, const void* coord, void* output, int batch, int channels, int dims,
                                const int* shape, int dtype, void* stream) {
  NdShape sh;
  int prod;
  if (!data || !coord || !output) return DK_ERR_BAD_ARGUMENT;
  int rc = nd_args(batch, channels, dims, shape, &sh, &prod);
  if (rc) return rc;
  DK_DISPATCH(dtype, nd_forward<T>(P_(T, data), P_(T, coord), M_(T, output), batch, channels, dims, prod, sh,
                                   (cudaStream_t)stream))
}

int dk_nd_linear_sample_backward_data(const void* grad_output, const void* coord, void* grad_data, int batch,
                                      int channels, int dims, const int* shape, int dtype, void* stream) {
  NdShape sh;
  int prod;
  if (!grad_output || !coord || !grad_data) return DK_ERR_BAD_ARGUMENT;
  int rc = nd_args(batch, channels, dims, shape, &sh, &prod);
  if (rc) return rc;
  DK_DISPATCH(dtype, nd_backward_data<T>(P_(T, grad_output), P_(T, coord), M_(T, grad_data), batch, channels, dims, prod,
                                         sh, (cudaStream_t)stream))
}

int dk_nd_linear_sample_backward_coord(const void* grad_output, const void* data, const void* coord,
                                       void* grad_coord_per_channel, int batch, int channels, int dims, const int* shape,
                                       int dtype, void* stream) {
  NdShape sh;
  int prod;
  if (!grad_output || !data || !coord || !grad_coord_per_channel) return DK_ERR_BAD_ARGUMENT;
  int rc = nd_args(batch, channels, dims, shape, &sh, &prod);
  if (rc) return rc;
  DK_DISPATCH(dtype, nd_backward_coord<T>(P_(T, grad_output), P_(T, data), P_(T, coord), M_(T, grad_coord_per_channel),
                                          batch, channels, dims, prod, sh, false, (cudaStream_t)stream))
}

int dk_nd_linear_sample_backward_coord_sum(const void* grad_output, const void* data, const void* coord, void* grad_coord,
                                           int batch, int channels, int dims, const int* shape, int dtype, void* stream) {
  NdShape sh;
  int prod;
  if (!grad_output || !data || !coord || !grad_coord) return DK_ERR_BAD_ARGUMENT;
  int rc = nd_args(batch, channels, dims, shape, &sh, &prod);
  if (rc) return rc;
  DK_DISPATCH(dtype, nd_backward_coord<T>(P_(T, grad_output), P_(T, data), P_(T, coord), M_(T, grad_coord), batch,
                                          channels, dims, prod, sh, true, (cudaStream_t)stream))
}

/* ---------------------------------------------------------------- fused global DK (1x1 depthwise) */

size_t dk_global_dk_backward_workspace_bytes(int batch, int channels, int dims) {
  if (batch <= 0 || channels <= 0 || dims <= 0) return 0;
  return align256(((size_t)2 * batch * channels + (size_t)batch * dims) * sizeof(float));
}

int dk_global_dk_forward(const void* input, const void* bank, const void* fc_weight, const void* fc_bias,
                         const void* tap_bias, void* output, void* pooled, void* raw_coord, void* coord, void* scale,
                         int batch, int channels, int plane_size, int dims, const int* shape, int dtype, void* stream) {
  NdShape sh;
  int prod;
  if (!input || !bank || !fc_weight || !fc_bias || !tap_bias || !output || !pooled || !raw_coord || !coord || !scale ||
      plane_size <= 0)
    return DK_ERR_BAD_ARGUMENT;
  int rc = nd_args(batch, channels, dims, shape, &sh, &prod);
  if (rc) return rc;
  DK_DISPATCH(dtype, global_dk_forward<T>(P_(T, input), P_(float, bank), P_(float, fc_weight), P_(float, fc_bias),
                                          P_(float, tap_bias), M_(T, output), M_(float, pooled), M_(float, raw_coord),
                                          M_(float, coord), M_(float, scale), batch, channels, plane_size, dims, prod, sh,
                                          (cudaStream_t)stream))
}

int dk_global_dk_backward(const void* grad_output, const void* input, const void* bank, const void* fc_weight,
                          const void* pooled, const void* raw_coord, const void* coord, const void* scale, void* grad_input,
                          void* grad_bank, void* grad_fc_weight, void* grad_fc_bias, int batch, int channels, int plane_size,
                          int dims, const int* shape, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  NdShape sh;
  int prod;
  if (!grad_output || !input || !bank || !fc_weight || !pooled || !raw_coord || !coord || !scale || plane_size <= 0)
    return DK_ERR_BAD_ARGUMENT;
  int rc = nd_args(batch, channels, dims, shape, &sh, &prod);
  if (rc) return rc;
  if (!workspace || workspace_bytes < dk_global_dk_backward_workspace_bytes(batch, channels, dims)) return DK_ERR_WORKSPACE;
  DK_DISPATCH(dtype, global_dk_backward<T>(P_(T, grad_output), P_(T, input), P_(float, bank), P_(float, fc_weight),
                                           P_(float, pooled), P_(float, raw_coord), P_(float, coord), P_(float, scale),
                                           M_(T, grad_input), M_(float, grad_bank), M_(float, grad_fc_weight),
                                           M_(float, grad_fc_bias), M_(float, workspace), batch, channels, plane_size, dims,
                                           prod, sh, (cudaStream_t)stream))
}

}  // extern "C"
