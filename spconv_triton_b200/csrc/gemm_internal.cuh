// Internal (non-ABI) interfaces between the GEMM translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "common.cuh"

namespace spc {

// out[rm, n] = sum_k sum_r src[pairs[k, rm], r] * w[n*s_wn + k*s_wk + r*s_wr] (+ bias[n]),
// rm = order ? order[slot] : slot.  CUDA-core kernel, any channel counts.
int gather_gemm_simt(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                     const int32_t* order, void* out, long long m_rows, int n_dim, int r_dim, int kv,
                     long long s_wk, long long s_wr, long long s_wn, int dtype, int out_dtype,
                     cudaStream_t st);

struct WgradSplit {
  int splits;
  int64_t rows_per_split;
  size_t bytes;  // fp32 partial sums [splits, c_out, kv, c_in]
};
WgradSplit wgrad_split(int64_t n_out, int c_in, int c_out, int kv);

int wgrad_simt(const void* feats, const void* gout, const int32_t* pair_fwd, void* dw, float* partial,
               int64_t n_out, int c_in, int c_out, int kv, int dtype, cudaStream_t st);

// tcgen05 kernels (gemm_tc.cu).  `transposed_weight` selects the input-gradient
// view of the KRSC weight.  Return SPC_ERR_UNSUPPORTED for shapes they do not take.
bool gather_gemm_tc_supported(int n_dim, int r_dim, int kv, int dtype, int out_dtype, int precision,
                              bool transposed_weight);
int gather_gemm_tc(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                   const int32_t* order, void* out, long long m_rows, int n_dim, int r_dim, int kv,
                   bool transposed_weight, int dtype, int out_dtype, int precision, cudaStream_t st);

// dw[e] = sum over splits of partial[s, e], added in split order (deterministic).
int wgrad_reduce(const float* partial, void* dw, long long elems, int splits, int dtype, cudaStream_t st);

// tcgen05 weight gradient (gemm_wgrad_tc.cu): fp32 partial tiles, to be followed by wgrad_reduce.
bool wgrad_tc_supported(int c_in, int c_out, int kv, int dtype);
WgradSplit wgrad_tc_split(int64_t n_out, int c_in, int c_out, int kv);
int wgrad_tc(const void* feats, const void* gout, const int32_t* pair_fwd, float* partial, int64_t n_out, int c_in,
             int c_out, int kv, int dtype, const WgradSplit& split, cudaStream_t st);

int* device_status_ptr();

// Variant of the tcgen05 kernel (gemm_tma.cu) whose weight slabs arrive by tiled TMA loads;
// the gathered feature rows are copied with cp.async.
bool gather_gemm_tma_supported(int n_dim, int r_dim, int kv, int dtype, int out_dtype, int precision,
                               bool transposed_weight);
int gather_gemm_tma(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                    const int32_t* pairs_rowmajor, const int32_t* order, void* out, long long src_rows, long long m_rows, int n_dim, int r_dim,
                    int kv, bool transposed_weight, int dtype, int out_dtype, int precision, cudaStream_t st);

}  // namespace spc
