// Several copies of the residual stream that every sublayer reads as one weighted sum and
// writes back through a small mixing matrix ("hyper-connections").
//
// With S streams x_1 .. x_S of a token (x[T, S, H], 32-bit), a sublayer q with the learned
// vectors a[S], b[S] and the matrix M[S, S] (indexed [from, to]) does
//   u   = sum_s a[s] x_s                      (read; the sublayer's norm follows)
//   y   = sublayer(norm(u))
//   x_t = sum_s M[s, t] x_s + b[t] y          (write, all streams at once from the old ones)
// Both kernels are 32-bit throughout.  The read kernel can apply an RMS norm to u on the way
// (out = u / sqrt(mean(u^2) + eps) * w, in the compute dtype) and zeroes the 32-bit buffer
// that the sublayer will add its output into, so a sublayer costs two launches beside its own.
#include "common.cuh"

using namespace ilb;

constexpr int kMaxStreams = 16;

// One block per token.  u is kept in shared memory between the sum and the norm.
template <typename TO>
__global__ void __launch_bounds__(256)
streams_read_kernel(const float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ w,
                    TO* __restrict__ normed, float* __restrict__ u_out, float* __restrict__ y_zero,
                    int width, int streams, float eps) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ float u[];
  __shared__ float scratch[33];
  __shared__ float coef[kMaxStreams];
  if (threadIdx.x < streams) coef[threadIdx.x] = a[threadIdx.x];
  __syncthreads();
  const float* row = x + (size_t)blockIdx.x * streams * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = coef[0] * row[i];
    for (int s = 1; s < streams; ++s) v = fmaf(coef[s], row[(size_t)s * width + i], v);
    u[i] = v;
    ss = fmaf(v, v, ss);
    if (u_out != nullptr) u_out[(size_t)blockIdx.x * width + i] = v;
    if (y_zero != nullptr) y_zero[(size_t)blockIdx.x * width + i] = 0.f;
  }
  if (normed == nullptr) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  TO* o = normed + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_float<TO>(u[i] * inv * w[i]);
}

// x: [T, S, H] 32-bit.  a: [S].  With `norm_weight` given, `normed` [T, H] (out_dtype) receives
// the RMS norm of u; `u_out` [T, H] 32-bit, if given, receives u itself (for a norm of another
// kind); `y_zero` [T, H] 32-bit, if given, is set to zero.
ILB_EXPORT int ilb_streams_read(const float* x, const float* a, const float* norm_weight, void* normed, int out_dtype,
                                float* u_out, float* y_zero, int n_tokens, int width, int streams, float eps,
                                cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && width > 0 && streams > 0 && streams <= kMaxStreams, "streams_read: bad sizes T=%d H=%d S=%d",
              n_tokens, width, streams);
  ILB_REQUIRE((norm_weight == nullptr) == (normed == nullptr), "streams_read: a norm needs its weight and its output");
  ILB_REQUIRE(normed == nullptr || eps > 0.f, "streams_read: eps must be positive");
  ILB_REQUIRE((size_t)width * 4 <= 160 * 1024, "streams_read: width %d does not fit shared memory", width);
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  const size_t smem = (size_t)width * sizeof(float);
  static OncePerDevice once_f, once_b;
  if (out_dtype == kF32 || normed == nullptr) {
    if (smem > 48 * 1024 && once_f.first() &&
        cudaFuncSetAttribute(streams_read_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) {
      once_f.forget();
      return fail("streams_read: cannot reserve shared memory");
    }
    ilb::launch(streams_read_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream, x, a, norm_weight, (float*)normed, u_out,
                y_zero, width, streams, eps);
  } else if (out_dtype == kBF16) {
    if (smem > 48 * 1024 && once_b.first() &&
        cudaFuncSetAttribute(streams_read_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) {
      once_b.forget();
      return fail("streams_read: cannot reserve shared memory");
    }
    ilb::launch(streams_read_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), smem, stream, x, a, norm_weight,
                (__nv_bfloat16*)normed, u_out, y_zero, width, streams, eps);
  } else {
    return fail("streams_read: unknown output dtype %d", out_dtype);
  }
  return check_launch("streams_read");
}

// In place on x[T, S, H]: every stream of a (token, feature) from the old values of all of them.
__global__ void __launch_bounds__(256)
streams_write_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                     const float* __restrict__ b, int width, int streams, size_t n) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float m[kMaxStreams * kMaxStreams];
  __shared__ float bo[kMaxStreams];
  for (int i = threadIdx.x; i < streams * streams; i += blockDim.x) m[i] = mix[i];
  if (threadIdx.x < streams) bo[threadIdx.x] = b[threadIdx.x];
  __syncthreads();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i % width);
    float* col = x + t * streams * width + c;
    float old[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < streams) old[s] = col[(size_t)s * width];
    const float yv = y[i];
#pragma unroll
    for (int to = 0; to < kMaxStreams; ++to) {
      if (to >= streams) break;
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < streams) v = fmaf(m[s * streams + to], old[s], v);
      col[(size_t)to * width] = fmaf(bo[to], yv, v);
    }
  }
}

// x[t, to, :] = sum_s mix[s, to] * x[t, s, :] + b[to] * y[t, :]
ILB_EXPORT int ilb_streams_write(float* x, const float* y, const float* mix, const float* b, int n_tokens, int width,
                                 int streams, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && width > 0 && streams > 0 && streams <= kMaxStreams, "streams_write: bad sizes");
  if (n_tokens == 0) return 0;
  const size_t n = (size_t)n_tokens * width;
  const int threads = 256;
  size_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ilb::launch(streams_write_kernel, dim3((int)blocks), dim3(threads), 0, stream, x, y, mix, b, width, streams, n);
  return check_launch("streams_write");
}

ILB_DEFINE_LAST_ERROR()
