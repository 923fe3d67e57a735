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
  const float* row = x + (size_t)blockIdx.x * streams * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = __ldg(a) * row[i];
    for (int s = 1; s < streams; ++s) v = fmaf(__ldg(a + s), row[(size_t)s * width + i], v);
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

// The same with the row in registers: S streams known at compile time, 16-byte accesses, every
// load of a thread in flight before the first sum (a thread holds kVecs pieces of four features).
// The sum of squares is added in the same order whatever the batch: it depends on the width alone.
constexpr int kVecs = 2;

template <typename TO, int S>
__global__ void __launch_bounds__(1024)
streams_read_vec_kernel(const float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ w,
                        TO* __restrict__ normed, float* __restrict__ u_out, float* __restrict__ y_zero, int width, float eps) {
  ilb::pdl_launch_dependents();
  float coef[S];
#pragma unroll
  for (int s = 0; s < S; ++s) coef[s] = __ldg(a + s);         // (weights: no earlier kernel writes them)
  const int n4 = width / 4;
  float4 g[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int j = threadIdx.x + i * blockDim.x;
    g[i] = (j < n4 && w != nullptr) ? __ldg(reinterpret_cast<const float4*>(w) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  ilb::pdl_wait();
  __shared__ float scratch[33];
  const float4* row = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * S * width);
  float4 v[kVecs][S];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int j = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int s = 0; s < S; ++s) v[i][s] = j < n4 ? row[(size_t)s * n4 + j] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float4 u[kVecs];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    u[i] = make_float4(coef[0] * v[i][0].x, coef[0] * v[i][0].y, coef[0] * v[i][0].z, coef[0] * v[i][0].w);
#pragma unroll
    for (int s = 1; s < S; ++s) {
      u[i].x = fmaf(coef[s], v[i][s].x, u[i].x); u[i].y = fmaf(coef[s], v[i][s].y, u[i].y);
      u[i].z = fmaf(coef[s], v[i][s].z, u[i].z); u[i].w = fmaf(coef[s], v[i][s].w, u[i].w);
    }
    ss = fmaf(u[i].x, u[i].x, ss); ss = fmaf(u[i].y, u[i].y, ss); ss = fmaf(u[i].z, u[i].z, ss); ss = fmaf(u[i].w, u[i].w, ss);
    const int j = threadIdx.x + i * blockDim.x;
    if (j < n4) {
      if (u_out != nullptr) reinterpret_cast<float4*>(u_out + (size_t)blockIdx.x * width)[j] = u[i];
      if (y_zero != nullptr) reinterpret_cast<float4*>(y_zero + (size_t)blockIdx.x * width)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (normed == nullptr) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  TO* o = normed + (size_t)blockIdx.x * width;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int j = threadIdx.x + i * blockDim.x;
    if (j >= n4) continue;
    const float p = u[i].x * inv * g[i].x, q = u[i].y * inv * g[i].y, r = u[i].z * inv * g[i].z, t = u[i].w * inv * g[i].w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(o)[j] = make_float4(p, q, r, t);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p, q), hi = __floats2bfloat162_rn(r, t);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(o)[j] = pk;
    }
  }
}

template <typename TO>
static bool launch_read_vec(const float* x, const float* a, const float* w, TO* normed, float* u_out, float* y_zero, int n_tokens,
                            int width, int streams, float eps, cudaStream_t stream) {
  int threads = (width / 4 + kVecs - 1) / kVecs;
  threads = (threads + 31) / 32 * 32;
#define ILB_READ(S_) ilb::launch(streams_read_vec_kernel<TO, S_>, dim3(n_tokens), dim3(threads), 0, stream, x, a, w, normed, u_out, y_zero, width, eps)
  switch (streams) {
    case 1: ILB_READ(1); return true;
    case 2: ILB_READ(2); return true;
    case 3: ILB_READ(3); return true;
    case 4: ILB_READ(4); return true;
    default: return false;
  }
#undef ILB_READ
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
  const bool vec = width % 4 == 0 && width >= 256 && width <= 4 * 1024 * kVecs && streams <= 4 && ((uintptr_t)x % 16 == 0) &&
                   ((uintptr_t)norm_weight % 16 == 0) && ((uintptr_t)normed % 16 == 0) && ((uintptr_t)u_out % 16 == 0) &&
                   ((uintptr_t)y_zero % 16 == 0);
  if (vec) {
    bool done;
    if (out_dtype == kBF16 && normed != nullptr)
      done = launch_read_vec<__nv_bfloat16>(x, a, norm_weight, (__nv_bfloat16*)normed, u_out, y_zero, n_tokens, width, streams, eps, stream);
    else if (out_dtype == kF32 || normed == nullptr)
      done = launch_read_vec<float>(x, a, norm_weight, (float*)normed, u_out, y_zero, n_tokens, width, streams, eps, stream);
    else
      return fail("streams_read: unknown output dtype %d", out_dtype);
    if (done) return check_launch("streams_read");
  }
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
    for (int s = 0; s < streams; ++s) old[s] = col[(size_t)s * width];
    const float yv = y[i];
    for (int to = 0; to < streams; ++to) {
      float v = 0.f;
      for (int s = 0; s < streams; ++s) v = fmaf(m[s * streams + to], old[s], v);
      col[(size_t)to * width] = fmaf(bo[to], yv, v);
    }
  }
}

// The same for up to four streams, known at compile time: the coefficients in registers, four
// features per thread with 16-byte accesses, the same sums in the same order.
template <int S>
__global__ void __launch_bounds__(256)
streams_write_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                         const float* __restrict__ b, int n4_row, size_t n4) {
  ilb::pdl_launch_dependents();
  float m[S][S], bo[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    bo[s] = __ldg(b + s);
#pragma unroll
    for (int t = 0; t < S; ++t) m[s][t] = __ldg(mix + s * S + t);
  }
  ilb::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const size_t t = i / n4_row;
  const int c = (int)(i % n4_row);
  float4* col = reinterpret_cast<float4*>(x) + t * S * n4_row + c;
  float4 old[S];
#pragma unroll
  for (int s = 0; s < S; ++s) old[s] = col[(size_t)s * n4_row];
  const float4 yv = reinterpret_cast<const float4*>(y)[i];
#pragma unroll
  for (int to = 0; to < S; ++to) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < S; ++s) {
      v.x = fmaf(m[s][to], old[s].x, v.x); v.y = fmaf(m[s][to], old[s].y, v.y);
      v.z = fmaf(m[s][to], old[s].z, v.z); v.w = fmaf(m[s][to], old[s].w, v.w);
    }
    col[(size_t)to * n4_row] = make_float4(fmaf(bo[to], yv.x, v.x), fmaf(bo[to], yv.y, v.y), fmaf(bo[to], yv.z, v.z), fmaf(bo[to], yv.w, v.w));
  }
}

// x[t, to, :] = sum_s mix[s, to] * x[t, s, :] + b[to] * y[t, :]
ILB_EXPORT int ilb_streams_write(float* x, const float* y, const float* mix, const float* b, int n_tokens, int width,
                                 int streams, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && width > 0 && streams > 0 && streams <= kMaxStreams, "streams_write: bad sizes");
  if (n_tokens == 0) return 0;
  const size_t n = (size_t)n_tokens * width;
  const int threads = 256;
  if (width % 4 == 0 && streams <= 4 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && (n / 4 + threads - 1) / threads <= 2147483647u) {
    const size_t n4 = n / 4;
    const dim3 grid((unsigned)((n4 + threads - 1) / threads));
    switch (streams) {
      case 1: ilb::launch(streams_write_vec_kernel<1>, grid, dim3(threads), 0, stream, x, y, mix, b, width / 4, n4); break;
      case 2: ilb::launch(streams_write_vec_kernel<2>, grid, dim3(threads), 0, stream, x, y, mix, b, width / 4, n4); break;
      case 3: ilb::launch(streams_write_vec_kernel<3>, grid, dim3(threads), 0, stream, x, y, mix, b, width / 4, n4); break;
      default: ilb::launch(streams_write_vec_kernel<4>, grid, dim3(threads), 0, stream, x, y, mix, b, width / 4, n4); break;
    }
    return check_launch("streams_write");
  }
  size_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ilb::launch(streams_write_kernel, dim3((int)blocks), dim3(threads), 0, stream, x, y, mix, b, width, streams, n);
  return check_launch("streams_write");
}

ILB_DEFINE_LAST_ERROR()
