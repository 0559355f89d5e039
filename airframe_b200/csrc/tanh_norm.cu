// The norm without statistics, y = tanh(alpha x) w + b (alpha a scalar, w and b vectors), alone and
// fused with the residual sum around it, and the re-entry of a repeated stretch of layers
// (x <- W [x; x0] + row).  Everything here is elementwise and 32-bit; the rows that feed matrix products
// leave in the compute dtype.
#include "common.cuh"

// y = tanh(alpha x) w + b with exact tanhf
__device__ __forceinline__ float tanh_norm_f32(float x, float alpha, float w, float b) { return tanhf(alpha * x) * w + b; }

// A term of a sum that may come as `n_parts` float partial sums (added in index order) or as one row of
// the compute dtype.
template <typename TA>
__device__ __forceinline__ float summed(const TA* a, int n_parts, size_t part_stride, size_t at) {
  float v = to_f32(a[at]);
  for (int p = 1; p < n_parts; ++p) v += to_f32(a[(size_t)p * part_stride + at]);
  return v;
}

// y[r] = tanh_norm(x[src(r)]); rows gathered by `rows` when given.
template <typename TY>
__global__ void __launch_bounds__(256)
tanh_norm_kernel(TY* __restrict__ y, const float* __restrict__ x, const float* __restrict__ w,
                 const float* __restrict__ b, float alpha, const int* __restrict__ rows, int hidden, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (at >= total) return;
  const size_t r = at / hidden;
  const int i = (int)(at - r * hidden);
  const float v = rows ? x[(size_t)rows[r] * hidden + i] : x[at];
  y[at] = from_f32<TY>(tanh_norm_f32(v, alpha, w[i], b[i]));
}

AF_EXPORT int af_tanh_norm(void* y, int y_dtype, const float* x, const float* w, const float* b, float alpha,
                           const int* rows, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && hidden > 0, "af_tanh_norm: bad sizes");
  const size_t total = (size_t)n_rows * hidden;
  const size_t blocks = (total + 255) / 256;
  AF_REQUIRE(blocks < (1ull << 31), "af_tanh_norm: too many rows");
  AF_DISPATCH_DTYPE(y_dtype, TY,
                    af_launch(tanh_norm_kernel<TY>, dim3((unsigned)blocks), dim3(256), 0, stream, (TY*)y, x, w, b, alpha,
                              rows, hidden, total));
  AF_CHECK_LAUNCH("af_tanh_norm");
}

// x += tanh_norm_post(a); then, when y is given, y = tanh_norm_next(x).  `a` may come as `n_parts`
// partial sums (float, [n_parts, rows, hidden]).  Four elements a thread where hidden % 4 == 0.
template <typename TA, typename TY, int V>
__global__ void __launch_bounds__(256)
add_tanh_norm_kernel(float* __restrict__ x, const TA* __restrict__ a, int n_parts, size_t part_stride,
                     const float* __restrict__ w_post, const float* __restrict__ b_post, float alpha_post,
                     TY* __restrict__ y, const float* __restrict__ w_next, const float* __restrict__ b_next,
                     float alpha_next, int hidden, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (at >= total) return;
  const int i = (int)(at % hidden);
  float xv[V];
  if (V == 4) {
    const float4 t = *reinterpret_cast<const float4*>(x + at);
    xv[0] = t.x, xv[1] = t.y, xv[2] = t.z, xv[3 % V] = t.w;
  } else {
    xv[0] = x[at];
  }
#pragma unroll
  for (int u = 0; u < V; ++u)
    xv[u] += tanh_norm_f32(summed(a, n_parts, part_stride, at + u), alpha_post, w_post[i + u], b_post[i + u]);
  if (V == 4) *reinterpret_cast<float4*>(x + at) = make_float4(xv[0], xv[1 % V], xv[2 % V], xv[3 % V]);
  else x[at] = xv[0];
  if (y == nullptr) return;
#pragma unroll
  for (int u = 0; u < V; ++u) y[at + u] = from_f32<TY>(tanh_norm_f32(xv[u], alpha_next, w_next[i + u], b_next[i + u]));
}

AF_EXPORT int af_add_tanh_norm(float* x, const void* a, int a_dtype, int n_parts, long long part_stride,
                               const float* w_post, const float* b_post, float alpha_post, void* y, int y_dtype,
                               const float* w_next, const float* b_next, float alpha_next, int n_rows, int hidden,
                               cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 1, "af_add_tanh_norm: bad sizes");
  AF_REQUIRE(a_dtype == AF_F32 || n_parts == 1, "af_add_tanh_norm: partial sums are float");
  AF_REQUIRE(y == nullptr || (w_next != nullptr && b_next != nullptr), "af_add_tanh_norm: a norm needs its weights");
  const size_t total = (size_t)n_rows * hidden;
  const bool vec = hidden % 4 == 0 && ((uintptr_t)x & 15) == 0;
  const size_t threads = vec ? total / 4 : total;
  const size_t blocks = (threads + 255) / 256;
  AF_REQUIRE(blocks < (1ull << 31), "af_add_tanh_norm: too many rows");
#define AF_ATN(TA, TY, V)                                                                                            \
  af_launch(add_tanh_norm_kernel<TA, TY, V>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (const TA*)a, n_parts, \
            (size_t)part_stride, w_post, b_post, alpha_post, (TY*)y, w_next, b_next, alpha_next, hidden, total)
  AF_DISPATCH_DTYPE(a_dtype, TA, AF_DISPATCH_DTYPE(y_dtype, TY, if (vec) AF_ATN(TA, TY, 4); else AF_ATN(TA, TY, 1)));
#undef AF_ATN
  AF_CHECK_LAUNCH("af_add_tanh_norm");
}

// out[r] = [a[r] | b[r]] in the compute dtype: the input rows of a product over two float streams.
// V elements a thread (4 where both widths divide by 4: a group then lies in one of the two streams).
template <typename T, int V>
__global__ void __launch_bounds__(256)
concat_cast_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, int ha, int hb,
                   size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (at >= total) return;
  const int wdt = ha + hb;
  const size_t r = at / wdt;
  const int i = (int)(at - r * wdt);
  const float* src = i < ha ? a + r * ha + i : b + r * hb + (i - ha);
  if (V == 4) {
    const float4 v = *reinterpret_cast<const float4*>(src);
    out[at] = from_f32<T>(v.x), out[at + 1] = from_f32<T>(v.y), out[at + 2] = from_f32<T>(v.z), out[at + 3] = from_f32<T>(v.w);
  } else {
    out[at] = from_f32<T>(*src);
  }
}

AF_EXPORT int af_concat_cast(void* out, int dtype, const float* a, const float* b, int n_rows, int ha, int hb,
                             cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && ha > 0 && hb > 0, "af_concat_cast: bad sizes");
  const size_t total = (size_t)n_rows * (ha + hb);
  const bool vec = ha % 4 == 0 && hb % 4 == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
  const size_t blocks = ((vec ? total / 4 : total) + 255) / 256;
  AF_REQUIRE(blocks < (1ull << 31), "af_concat_cast: too many rows");
  if (vec) {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(concat_cast_kernel<T, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, a, b, ha, hb,
                                total));
  } else {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(concat_cast_kernel<T, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, a, b, ha, hb,
                                total));
  }
  AF_CHECK_LAUNCH("af_concat_cast");
}

// x = (the sum of the partial sums z) + row, for every row of x; then, when y is given, y = tanh_norm(x).
template <typename TZ, typename TY>
__global__ void __launch_bounds__(256)
set_sum_row_kernel(float* __restrict__ x, const TZ* __restrict__ z, int n_parts, size_t part_stride,
                   const float* __restrict__ row, TY* __restrict__ y, const float* __restrict__ w,
                   const float* __restrict__ b, float alpha, int hidden, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (at >= total) return;
  const int i = (int)(at % hidden);
  const float v = summed(z, n_parts, part_stride, at) + row[i];
  x[at] = v;
  if (y != nullptr) y[at] = from_f32<TY>(tanh_norm_f32(v, alpha, w[i], b[i]));
}

AF_EXPORT int af_set_sum_row(float* x, const void* z, int z_dtype, int n_parts, long long part_stride, const float* row,
                             void* y, int y_dtype, const float* w, const float* b, float alpha, int n_rows, int hidden,
                             cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 1, "af_set_sum_row: bad sizes");
  AF_REQUIRE(z_dtype == AF_F32 || n_parts == 1, "af_set_sum_row: partial sums are float");
  AF_REQUIRE(y == nullptr || (w != nullptr && b != nullptr), "af_set_sum_row: a norm needs its weights");
  const size_t total = (size_t)n_rows * hidden;
  const size_t blocks = (total + 255) / 256;
  AF_REQUIRE(blocks < (1ull << 31), "af_set_sum_row: too many rows");
  AF_DISPATCH_DTYPE(z_dtype, TZ, AF_DISPATCH_DTYPE(y_dtype, TY,
                    af_launch(set_sum_row_kernel<TZ, TY>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (const TZ*)z,
                              n_parts, (size_t)part_stride, row, (TY*)y, w, b, alpha, hidden, total)));
  AF_CHECK_LAUNCH("af_set_sum_row");
}
