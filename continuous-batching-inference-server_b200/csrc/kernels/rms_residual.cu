// Root-mean-square norms around the residual stream, in 32-bit arithmetic whatever the storage types.
//
//   add_rmsnorm: what a part produced is (optionally) normalised itself, added to the residual stream, and the
//   stream's row is normalised for the next part, all in one pass over the row:
//     d = delta[s,:] (+ delta_bias)                                           what the part before left
//     if post_w: d = d / sqrt(mean(d^2) + post_eps) * (post_offset + post_w)   a norm AFTER the part
//     d = d * delta_scale                                                      a constant on everything that is added
//     v = x[s,:] + d;  x[s,:] = v                                             the stream moves on (32-bit)
//     out[r,:] = v / sqrt(mean(v^2) + eps) * (offset + w)                      the norm BEFORE the next part
//   offset 1 is for weights stored around zero, offset 0 for weights stored as they are applied.  With `rows` only
//   those rows are produced and x is left as it is (the rows whose logits are wanted, before the head).
#include "common.cuh"

namespace cbis {

// One block per output row r; source row s = rows ? rows[r] : r.  The row and the delta wait in shared memory
// (2 d floats) between the passes, so x and delta are read once.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* x, const TD* delta, int delta_ld, const float* __restrict__ delta_bias,
                                   const float* __restrict__ post_w, float post_eps, float post_offset,
                                   const float* __restrict__ w, float eps, float offset, TO* out, const int* rows,
                                   int d, float delta_scale) {
  extern __shared__ float smem[];
  float* row = smem;           // d floats
  float* dl = smem + d;        // d floats
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* xrow = x + (size_t)s * d;
  const TD* drow = delta ? delta + (size_t)s * delta_ld : nullptr;
  float dscale = 1.f;
  if (drow) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      float v = to_f32(drow[c]);
      if (delta_bias) v += delta_bias[c];
      dl[c] = v;
      ss += v * v;
    }
    if (post_w) dscale = 1.0f / sqrtf(block_sum(ss, red) / (float)d + post_eps);
    dscale *= delta_scale;
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = xrow[c];
    if (drow) v += post_w ? dl[c] * dscale * (post_offset + post_w[c]) : dl[c] * dscale;
    row[c] = v;
    ss += v * v;
  }
  const float inv = w ? 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps) : 1.f;      // no weight: the rows go on as they are
  const bool write_x = rows == nullptr && drow != nullptr;
  TO* orow = out ? out + (size_t)r * d : nullptr;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = row[c];
    if (write_x) xrow[c] = v;
    if (orow) from_f32(orow[c], w ? v * inv * (offset + w[c]) : v);
  }
}

// The same for widths that are a multiple of 4 and at most 128 * 4 * NV: the row and the delta stay in registers (NV
// float4 each per thread, 128 threads a row), every access is 16 bytes wide, the weights are fetched before the
// kernel waits for its predecessor.
template <typename TT>
__device__ __forceinline__ float4 ld4(const TT* p);
template <>
__device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&a);
  r.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}

template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(128)
add_rmsnorm_reg_kernel(float* x, const TD* delta, int delta_ld, const float* __restrict__ delta_bias,
                       const float* __restrict__ post_w, float post_eps, float post_offset, const float* __restrict__ w,
                       float eps, float offset, TO* out, const int* rows, int d, float delta_scale) {
  __shared__ float red[33];
  pdl_trigger();
  const int nvec = d >> 2;
  float4 wv[NV], pw[NV], db[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * 128;
    wv[i] = pw[i] = db[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < nvec) {
      if (w) wv[i] = *reinterpret_cast<const float4*>(w + 4 * c);
      if (post_w) pw[i] = *reinterpret_cast<const float4*>(post_w + 4 * c);
      if (delta_bias) db[i] = *reinterpret_cast<const float4*>(delta_bias + 4 * c);
    }
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* xrow = x + (size_t)s * d;
  const TD* drow = delta ? delta + (size_t)s * delta_ld : nullptr;
  float4 v[NV], dl[NV];
  float ssd = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * 128;
    v[i] = dl[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < nvec) {
      v[i] = *reinterpret_cast<const float4*>(xrow + 4 * c);
      if (drow) {
        const float4 t = ld4<TD>(drow + 4 * c);
        dl[i] = make_float4(t.x + db[i].x, t.y + db[i].y, t.z + db[i].z, t.w + db[i].w);
        ssd += (dl[i].x * dl[i].x + dl[i].y * dl[i].y) + (dl[i].z * dl[i].z + dl[i].w * dl[i].w);
      }
    }
  }
  float dscale = 1.f;
  if (drow && post_w) dscale = 1.0f / sqrtf(block_sum(ssd, red) / (float)d + post_eps);
  dscale *= delta_scale;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (threadIdx.x + i * 128 < nvec) {
      if (drow) {
        if (post_w) {
          v[i].x += dl[i].x * dscale * (post_offset + pw[i].x);
          v[i].y += dl[i].y * dscale * (post_offset + pw[i].y);
          v[i].z += dl[i].z * dscale * (post_offset + pw[i].z);
          v[i].w += dl[i].w * dscale * (post_offset + pw[i].w);
        } else {
          v[i].x += dl[i].x * dscale; v[i].y += dl[i].y * dscale; v[i].z += dl[i].z * dscale; v[i].w += dl[i].w * dscale;
        }
      }
      ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  const float inv = w ? 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps) : 1.f;      // no weight: the rows go on as they are
  const bool write_x = rows == nullptr && drow != nullptr;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * 128;
    if (c < nvec) {
      if (write_x) *reinterpret_cast<float4*>(xrow + 4 * c) = v[i];
      if (out) {
        float4 o = v[i];
        if (w) o = make_float4(o.x * inv * (offset + wv[i].x), o.y * inv * (offset + wv[i].y), o.z * inv * (offset + wv[i].z),
                               o.w * inv * (offset + wv[i].w));
        st4(out + (size_t)r * d + 4 * c, o);
      }
    }
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_rms_residual_max_width() { return (200 * 1024 / 4 - 64) / 2; }

// x: 32-bit [*, d]; delta (may be null): [*, delta_ld] of delta_dtype; out (may be null): [n, d] of out_dtype.
CBIS_EXPORT int cbis_add_rmsnorm(float* x, const void* delta, int delta_ld, int delta_dtype, const float* delta_bias,
                                 const float* post_w, float post_eps, float post_offset, const float* w, float eps,
                                 float offset, void* out, int out_dtype, const int* rows, int n, int d, void* stream,
                                 float delta_scale) {
  if (n <= 0) return CBIS_OK;
  if (d <= 0 || d > cbis_rms_residual_max_width()) return CBIS_ERR_BAD_SIZE;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  const size_t smem = (size_t)2 * d * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
#define CBIS_ARN(TD, TO)                                                                                              \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    return (int)launch_pdl(add_rmsnorm_kernel<TD, TO>, dim3(n), dim3(threads), smem, st, x, (const TD*)delta, delta_ld, \
                           delta_bias, post_w, post_eps, post_offset, w, eps, offset, (TO*)out, rows, d, delta_scale); \
  } while (0)
  const int dd = delta ? delta_dtype : CBIS_F32;
  // rows in registers where every piece is 16 bytes wide and aligned
  const int esz_d = dd == CBIS_F32 ? 4 : 2, esz_o = out_dtype == CBIS_F32 ? 4 : 2;
  const bool reg = d % 4 == 0 && d <= 128 * 4 * 8 && !((uintptr_t)x & 15) && !((uintptr_t)w & 15) && !((uintptr_t)post_w & 15) &&
                   !((uintptr_t)delta_bias & 15) && (!delta || (!((uintptr_t)delta & (4 * esz_d - 1)) && delta_ld % 4 == 0)) &&
                   (!out || !((uintptr_t)out & (4 * esz_o - 1)));
#define CBIS_ARN_REG(TD, TO, NV)                                                                                       \
  return (int)launch_pdl(add_rmsnorm_reg_kernel<TD, TO, NV>, dim3(n), dim3(128), 0, st, x, (const TD*)delta, delta_ld, \
                         delta_bias, post_w, post_eps, post_offset, w, eps, offset, (TO*)out, rows, d, delta_scale)
#define CBIS_ARN_PICK(TD, TO)                 \
  do {                                        \
    if (d <= 512) CBIS_ARN_REG(TD, TO, 1);    \
    if (d <= 1024) CBIS_ARN_REG(TD, TO, 2);   \
    if (d <= 2048) CBIS_ARN_REG(TD, TO, 4);   \
    CBIS_ARN_REG(TD, TO, 8);                  \
  } while (0)
  if (reg) {
    if (dd == CBIS_F32 && out_dtype == CBIS_F32) CBIS_ARN_PICK(float, float);
    if (dd == CBIS_F32 && out_dtype == CBIS_BF16) CBIS_ARN_PICK(float, __nv_bfloat16);
    if (dd == CBIS_BF16 && out_dtype == CBIS_BF16) CBIS_ARN_PICK(__nv_bfloat16, __nv_bfloat16);
    if (dd == CBIS_BF16 && out_dtype == CBIS_F32) CBIS_ARN_PICK(__nv_bfloat16, float);
  }
#undef CBIS_ARN_PICK
#undef CBIS_ARN_REG
  if (dd == CBIS_F32 && out_dtype == CBIS_F32) CBIS_ARN(float, float);
  if (dd == CBIS_F32 && out_dtype == CBIS_BF16) CBIS_ARN(float, __nv_bfloat16);
  if (dd == CBIS_BF16 && out_dtype == CBIS_BF16) CBIS_ARN(__nv_bfloat16, __nv_bfloat16);
  if (dd == CBIS_BF16 && out_dtype == CBIS_F32) CBIS_ARN(__nv_bfloat16, float);
#undef CBIS_ARN
  return CBIS_ERR_BAD_DTYPE;
}
