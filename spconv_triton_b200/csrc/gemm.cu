// C-ABI entry points of the implicit gather-GEMM and the choice between the
// tcgen05 kernels and the CUDA-core kernels.
#include <algorithm>

#include "common.cuh"
#include "gemm_internal.cuh"

using namespace spc;

namespace {

// The tensor-core kernels take 16-bit inputs always and fp32 inputs only when
// the caller allows TF32; IEEE fp32 stays on the CUDA cores.
bool want_tc(int path, int n_dim, int r_dim, int kv, int dtype, int out_dtype, int precision, bool transposed,
             int* status) {
  *status = SPC_OK;
  const bool ok = gather_gemm_tc_supported(n_dim, r_dim, kv, dtype, out_dtype, precision, transposed);
  if (path == SPC_GEMM_SIMT) return false;
  if (path == SPC_GEMM_TCGEN05) {
    if (!ok) *status = fail(SPC_ERR_UNSUPPORTED, "tcgen05 path does not take this shape/dtype "
                            "(n=%d r=%d kv=%d dtype=%d precision=%d)", n_dim, r_dim, kv, dtype, precision);
    return ok;
  }
  return ok;
}

}  // namespace

extern "C" int spc_conv_forward_needs_colmajor(int c_in, int c_out, int kv, int dtype, int out_dtype, int precision,
                                               int path) {
  const bool tma = path != SPC_GEMM_SIMT && path != SPC_GEMM_TCGEN05_CPASYNC &&
                   gather_gemm_tc_supported(c_out, c_in, kv, dtype, out_dtype, precision, false) &&
                   gather_gemm_tma_supported(c_out, c_in, kv, dtype, out_dtype, precision, false);
  return tma ? 0 : 1;
}

extern "C" int spc_conv_forward(const void* features, const void* weight, const void* bias,
                                const int32_t* pair_fwd, const int32_t* pair_fwd_rowmajor,
                                const int32_t* mask_argsort, void* out,
                                int64_t n_in, int64_t n_out, int c_in, int c_out, int kv, int dtype,
                                int out_dtype, int precision, int path, const float* out_scale,
                                const float* out_shift, int act, float act_alpha, void* stream) {
  return spc_conv_forward_residual(features, weight, bias, pair_fwd, pair_fwd_rowmajor, mask_argsort, out, n_in, n_out,
                                   c_in, c_out, kv, dtype, out_dtype, precision, path, out_scale, out_shift, act,
                                   act_alpha, nullptr, stream);
}

extern "C" int spc_conv_forward_residual(const void* features, const void* weight, const void* bias,
                                         const int32_t* pair_fwd, const int32_t* pair_fwd_rowmajor,
                                         const int32_t* mask_argsort, void* out, int64_t n_in, int64_t n_out,
                                         int c_in, int c_out, int kv, int dtype, int out_dtype, int precision,
                                         int path, const float* out_scale, const float* out_shift, int act,
                                         float act_alpha, const void* residual, void* stream) {
  if (!features || !weight || !out || n_in < 0 || n_out < 0 || c_in <= 0 || c_out <= 0 || kv <= 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_forward: bad arguments");
  if (!pair_fwd && (!pair_fwd_rowmajor ||
                    spc_conv_forward_needs_colmajor(c_in, c_out, kv, dtype, out_dtype, precision, path)))
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_forward: this layer reads the column-major table");
  if ((out_scale == nullptr) != (out_shift == nullptr))
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_forward: out_scale and out_shift go together");
  if (n_out == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Epilogue epi;
  epi.bias = bias; epi.scale = out_scale; epi.shift = out_shift; epi.act = act; epi.alpha = act_alpha;
  epi.residual = residual;
  if (residual != nullptr && (reinterpret_cast<uintptr_t>(residual) & 15u) != 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_forward: the residual must be 16-byte aligned");
  int status;
  if (want_tc(path, c_out, c_in, kv, dtype, out_dtype, precision, false, &status)) {
    if (path != SPC_GEMM_TCGEN05_CPASYNC &&
        gather_gemm_tma_supported(c_out, c_in, kv, dtype, out_dtype, precision, false))
      return gather_gemm_tma(features, weight, epi, pair_fwd, pair_fwd_rowmajor, mask_argsort, out, n_in, n_out, c_out, c_in, kv,
                             /*transposed_weight=*/false, dtype, out_dtype, precision, st);
    return gather_gemm_tc(features, weight, epi, pair_fwd, mask_argsort, out, n_out, c_out, c_in, kv,
                          /*transposed_weight=*/false, dtype, out_dtype, precision, st);
  }
  if (status != SPC_OK) return status;
  // weight[n, k, c]: reduction index c has stride 1, output channel n stride kv*c_in.
  return gather_gemm_simt(features, weight, epi, pair_fwd, mask_argsort, out, n_out, c_out, c_in, kv,
                          /*s_wk=*/c_in, /*s_wr=*/1, /*s_wn=*/static_cast<long long>(kv) * c_in, dtype,
                          out_dtype, st);
}

extern "C" int spc_conv_backward_input(const void* grad_out, const void* weight, const int32_t* pair_bwd,
                                       const int32_t* pair_bwd_rowmajor, const int32_t* mask_argsort, void* din, int64_t n_in, int64_t n_out,
                                       int c_in, int c_out, int kv, int dtype, int precision, int path,
                                       void* stream) {
  if (!grad_out || !weight || !pair_bwd || !din || n_in < 0 || n_out < 0 || c_in <= 0 || c_out <= 0 || kv <= 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_backward_input: bad arguments");
  if (n_in == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int status;
  if (want_tc(path, c_in, c_out, kv, dtype, dtype, precision, true, &status)) {
    if (path != SPC_GEMM_TCGEN05_CPASYNC && gather_gemm_tma_supported(c_in, c_out, kv, dtype, dtype, precision, true))
      return gather_gemm_tma(grad_out, weight, Epilogue{}, pair_bwd, pair_bwd_rowmajor, mask_argsort, din, n_out, n_in, c_in, c_out, kv,
                             /*transposed_weight=*/true, dtype, dtype, precision, st);
    return gather_gemm_tc(grad_out, weight, Epilogue{}, pair_bwd, mask_argsort, din, n_in, c_in, c_out, kv,
                          /*transposed_weight=*/true, dtype, dtype, precision, st);
  }
  if (status != SPC_OK) return status;
  // output channel is c (stride 1), reduction index is n (stride kv*c_in).
  return gather_gemm_simt(grad_out, weight, Epilogue{}, pair_bwd, mask_argsort, din, n_in, c_in, c_out, kv,
                          /*s_wk=*/c_in, /*s_wr=*/static_cast<long long>(kv) * c_in, /*s_wn=*/1, dtype, dtype,
                          st);
}

extern "C" size_t spc_conv_backward_weight_workspace_bytes(int64_t n_out, int c_in, int c_out, int kv) {
  if (n_out < 0 || c_in <= 0 || c_out <= 0 || kv <= 0) return 0;
  // enough for whichever kernel the call ends up using
  return std::max(wgrad_split(n_out, c_in, c_out, kv).bytes, wgrad_tc_split(n_out, c_in, c_out, kv).bytes);
}

extern "C" int spc_conv_backward_weight(const void* features, const void* grad_out, const int32_t* pair_fwd,
                                        void* dweight, void* workspace, size_t workspace_bytes, int64_t n_in,
                                        int64_t n_out, int c_in, int c_out, int kv, int dtype, int precision,
                                        int path, void* stream) {
  (void)n_in;
  (void)precision;
  if (!features || !grad_out || !pair_fwd || !dweight || n_out < 0 || c_in <= 0 || c_out <= 0 || kv <= 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_backward_weight: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_out == 0) {
    SPC_CUDA_OK(cudaMemsetAsync(dweight, 0, static_cast<size_t>(c_out) * kv * c_in * dtype_size(dtype), st));
    return SPC_OK;
  }
  if (path != SPC_GEMM_SIMT && wgrad_tc_supported(c_in, c_out, kv, dtype)) {
    const WgradSplit ts = wgrad_tc_split(n_out, c_in, c_out, kv);
    if (!workspace || workspace_bytes < ts.bytes)
      return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "conv_backward_weight: workspace %zu < %zu bytes", workspace_bytes,
                  ts.bytes);
    const int rc = wgrad_tc(features, grad_out, pair_fwd, static_cast<float*>(workspace), n_out, c_in, c_out, kv,
                            dtype, ts, st);
    if (rc != SPC_OK) return rc;
    return wgrad_reduce(static_cast<const float*>(workspace), dweight, static_cast<long long>(c_out) * kv * c_in,
                        ts.splits, dtype, st);
  }
  if (path == SPC_GEMM_TCGEN05)
    return fail(SPC_ERR_UNSUPPORTED, "conv_backward_weight: the tcgen05 kernel does not take this shape/dtype "
                "(c_in=%d c_out=%d dtype=%d)", c_in, c_out, dtype);
  const WgradSplit s = wgrad_split(n_out, c_in, c_out, kv);
  if (!workspace || workspace_bytes < s.bytes)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "conv_backward_weight: workspace %zu < %zu bytes", workspace_bytes,
                s.bytes);
  return wgrad_simt(features, grad_out, pair_fwd, dweight, static_cast<float*>(workspace), n_out, c_in, c_out,
                    kv, dtype, st);
}
