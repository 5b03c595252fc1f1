// Housekeeping entry points of the C ABI: version, error text, shape formulas.
#include <atomic>

#include "common.cuh"

namespace spc {
char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
static std::atomic<long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace spc

using namespace spc;

extern "C" int spc_version(void) { return 100; }

extern "C" const char* spc_last_error(void) { return error_buffer(); }

extern "C" long long spc_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int spc_conv_output_size(int ndim, const int32_t* in_shape, const int32_t* ksize,
                                    const int32_t* stride, const int32_t* padding, const int32_t* dilation,
                                    int32_t* out_shape) {
  if (ndim < 1 || !in_shape || !ksize || !stride || !padding || !dilation || !out_shape)
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_output_size: bad arguments");
  for (int i = 0; i < ndim; ++i) {
    if (ksize[i] == -1) {
      out_shape[i] = 1;
      continue;
    }
    if (stride[i] <= 0) return fail(SPC_ERR_INVALID_ARGUMENT, "conv_output_size: stride must be positive");
    const long long num = static_cast<long long>(in_shape[i]) + 2ll * padding[i] -
                          static_cast<long long>(dilation[i]) * (ksize[i] - 1) - 1;
    // floor division, as Python's // does for negative numerators
    long long q = num / stride[i];
    if ((num % stride[i] != 0) && ((num < 0) != (stride[i] < 0))) --q;
    out_shape[i] = static_cast<int32_t>(q + 1);
  }
  return SPC_OK;
}

extern "C" int spc_deconv_output_size(int ndim, const int32_t* in_shape, const int32_t* ksize,
                                      const int32_t* stride, const int32_t* padding, const int32_t* dilation,
                                      const int32_t* out_padding, int32_t* out_shape) {
  (void)dilation;  // the reference's formula does not use it
  if (ndim < 1 || !in_shape || !ksize || !stride || !padding || !out_padding || !out_shape)
    return fail(SPC_ERR_INVALID_ARGUMENT, "deconv_output_size: bad arguments");
  for (int i = 0; i < ndim; ++i) {
    if (ksize[i] == -1) return fail(SPC_ERR_INVALID_ARGUMENT, "deconv don't support kernel_size < 0");
    out_shape[i] = (in_shape[i] - 1) * stride[i] - 2 * padding[i] + ksize[i] + out_padding[i];
  }
  return SPC_OK;
}
