// Rotary positions and a gate per head, in 32-bit arithmetic whatever the storage type.
//
//   rope_rows: in every row r (position p = positions[r]) and every head, `dims` entries starting at a column are
//   rotated in pairs: entry i with entry i + dims/2 ("rotate half"), by the angle p * base^(-2 i / dims):
//     (u, v) -> (u cos a - v sin a, v cos a + u sin a).
//   With `neighbours` the pairs are the entries 2i and 2i + 1 instead; `length` multiplies cosine and sine (a rotation
//   that also stretches).  With `keep` >= 0 the heads from `keep_head0` on are ALSO written as they came, unrotated,
//   at dst column keep + (head - keep_head0) * width (a mixer whose values are its keys before the rotation).
//   Source and destination may be different buffers with different strides between heads (a head's rotated part is
//   moved to its place among the columns the attention kernel reads); entries beyond `dims` up to `width` are copied.
//   head_gate_mul: out[r, h, :] = x[r, h, :] * sigmoid(gate[r, h]), one number per row and head.
//   qk_prepare: what stands between a projection q | k | v and attention, in place, one pass over a row: a
//   root-mean-square norm over ALL of q at once and over ALL of k at once (weights as wide as the projections, not one
//   per head), then the rotation of every head of q and k, and values blended with another layer's values of the same
//   token: v <- (1 - lambda) v + lambda v_other.  Each of the three steps is optional.
//   blend_rows: the last of them alone.
#include "common.cuh"

namespace cbis {

// grid (rows); a thread takes pairs (head, i).  Angles in 32-bit from the integer position: a = p * f_i with the
// frequencies f_i = base^(-2 i / dims) handed in as a table (made on the host in 64-bit, rounded once); sincosf keeps
// its full range reduction (no fast-math).
template <typename TT>
__global__ void rope_rows_kernel(const TT* src, int src_ld, int src_col0, int src_head_stride, TT* dst, int dst_ld,
                                 int dst_col0, int dst_head_stride, const int* positions, int heads, int width, int dims,
                                 const float* __restrict__ freqs, int neighbours, float length, int keep, int keep_head0) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float p = (float)positions[r];
  const int half = dims / 2;
  const TT* s0 = src + (size_t)r * src_ld + src_col0;
  TT* d0 = dst + (size_t)r * dst_ld + dst_col0;
  const int per_head = half + (width - dims);      // pairs, then entries that pass unchanged
  for (int u = threadIdx.x; u < heads * per_head; u += blockDim.x) {
    const int h = u / per_head, i = u % per_head;
    const TT* sh = s0 + (size_t)h * src_head_stride;
    TT* dh = d0 + (size_t)h * dst_head_stride;
    TT* kp = (keep >= 0 && h >= keep_head0) ? dst + (size_t)r * dst_ld + keep + (size_t)(h - keep_head0) * width : nullptr;
    if (i < half) {
      float sn, cs;
      sincosf(p * freqs[i], &sn, &cs);
      const int c0 = neighbours ? 2 * i : i, c1 = neighbours ? 2 * i + 1 : i + half;
      const TT ra = sh[c0], rb = sh[c1];
      const float a = to_f32(ra), b = to_f32(rb);
      cs *= length;
      sn *= length;
      if (kp) {           // before the rotated values are stored: source and destination may be one buffer
        kp[c0] = ra;
        kp[c1] = rb;
      }
      from_f32(dh[c0], a * cs - b * sn);
      from_f32(dh[c1], b * cs + a * sn);
    } else {
      const int c = dims + (i - half);
      const TT v = sh[c];
      if (kp) kp[c] = v;
      dh[c] = v;
    }
  }
}

// grid over elements; x, out: [rows, heads * width]; gate: [rows, gate_ld] with the heads' numbers at gate_col0...
template <typename TT, typename TG>
__global__ void head_gate_mul_kernel(const TT* x, int x_ld, const TG* gate, int gate_ld, TT* out, int out_ld, int rows,
                                     int heads, int width) {
  pdl_trigger();
  pdl_wait();
  const size_t n = (size_t)heads * width, total = (size_t)rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n;
    const int c = (int)(i % n);
    const float g = sigmoid_f32(to_f32(gate[r * gate_ld + c / width]));
    from_f32(out[r * out_ld + c], to_f32(x[r * x_ld + c]) * g);
  }
}

// One block per row.  q and k wait in shared memory (d_q + d_k floats) between the sums of squares and the rotation;
// a value is rounded once, after norm, weight and rotation.
template <typename TT>
__global__ void qk_prepare_kernel(TT* buf, int ld, int q_off, int q_heads, int k_off, int k_heads, int width,
                                  const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                  const int* positions, const float* __restrict__ freqs, int dims, int v_off, int d_v,
                                  const TT* v_other, int v_other_ld, float lambda) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  TT* b = buf + (size_t)r * ld;
  const int d_q = q_heads * width, d_k = k_heads * width;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < d_q + d_k; c += blockDim.x) {
    const float v = to_f32(c < d_q ? b[q_off + c] : b[k_off + c - d_q]);
    row[c] = v;
    if (c < d_q) sq += v * v;
    else sk += v * v;
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (q_w) inv_q = 1.0f / sqrtf(block_sum(sq, red) / (float)d_q + eps);
  if (k_w) inv_k = 1.0f / sqrtf(block_sum(sk, red) / (float)d_k + eps);
  __syncthreads();
  const float p = (float)positions[r];
  const int half = dims / 2, per_head = half + (width - dims);      // pairs, then entries that pass unrotated
  for (int u = threadIdx.x; u < (q_heads + k_heads) * per_head; u += blockDim.x) {
    const int h = u / per_head, i = u % per_head;
    const bool is_q = h < q_heads;
    const int c0 = is_q ? h * width : (h - q_heads) * width;       // the head's first column within its projection
    const float* src = row + (is_q ? 0 : d_q) + c0;
    const float* w = is_q ? q_w : k_w;
    const float inv = is_q ? inv_q : inv_k;
    TT* dst = b + (is_q ? q_off : k_off) + c0;
    if (i < half) {
      float x0 = src[i] * inv, x1 = src[i + half] * inv;
      if (w) {
        x0 *= w[c0 + i];
        x1 *= w[c0 + i + half];
      }
      float sn, cs;
      sincosf(p * freqs[i], &sn, &cs);
      from_f32(dst[i], x0 * cs - x1 * sn);
      from_f32(dst[i + half], x1 * cs + x0 * sn);
    } else {
      const int c = dims + (i - half);
      float x0 = src[c] * inv;
      if (w) x0 *= w[c0 + c];
      from_f32(dst[c], x0);
    }
  }
  if (v_other) {
    const TT* o = v_other + (size_t)r * v_other_ld;
    for (int c = threadIdx.x; c < d_v; c += blockDim.x)
      from_f32(b[v_off + c], (1.0f - lambda) * to_f32(b[v_off + c]) + lambda * to_f32(o[c]));
  }
}

// out[r, c] = (1 - lambda) a[r, c] + lambda b[r, c]
template <typename TT>
__global__ void blend_rows_kernel(const TT* a, int a_ld, const TT* b, int b_ld, TT* out, int out_ld, float lambda,
                                  int rows, int n) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n;
    const int c = (int)(i % n);
    from_f32(out[r * out_ld + c], (1.0f - lambda) * to_f32(a[r * a_ld + c]) + lambda * to_f32(b[r * b_ld + c]));
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_qk_prepare_max_width() { return 200 * 1024 / 4 - 64; }

// buf [rows, ld] of the compute type, changed in place: q at columns q_off.. (q_heads x width), k at k_off..
// (k_heads x width), v at v_off.. (d_v).  q_w / k_w (may be null): the norms' weights, q_heads * width and
// k_heads * width wide; freqs (null with dims 0): dims / 2 numbers; v_other (may be null): [rows, v_other_ld].
CBIS_EXPORT int cbis_qk_prepare(void* buf, int ld, int q_off, int q_heads, int k_off, int k_heads, int width,
                                const float* q_w, const float* k_w, float eps, const int* positions, const float* freqs,
                                int dims, int v_off, int d_v, const void* v_other, int v_other_ld, float lambda, int rows,
                                int dtype, void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (q_heads < 0 || k_heads < 0 || width <= 0 || dims < 0 || dims > width || dims % 2 || (dims > 0 && !freqs))
    return CBIS_ERR_BAD_SIZE;
  const long long n = (long long)(q_heads + k_heads) * width;
  if (n > cbis_qk_prepare_max_width()) return CBIS_ERR_BAD_SIZE;
  const size_t smem = (size_t)n * sizeof(float);
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  cudaStream_t st = (cudaStream_t)stream;
#define CBIS_QKP(TT)                                                                                                  \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(qk_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    return (int)launch_pdl(qk_prepare_kernel<TT>, dim3(rows), dim3(threads), smem, st, (TT*)buf, ld, q_off, q_heads,  \
                           k_off, k_heads, width, q_w, k_w, eps, positions, freqs, dims, v_off, d_v,                  \
                           (const TT*)v_other, v_other_ld, lambda);                                                   \
  } while (0)
  if (dtype == CBIS_F32) CBIS_QKP(float);
  if (dtype == CBIS_BF16) CBIS_QKP(__nv_bfloat16);
#undef CBIS_QKP
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_blend_rows(const void* a, int a_ld, const void* b, int b_ld, void* out, int out_ld, float lambda,
                                int rows, int n, int dtype, void* stream) {
  if (rows <= 0 || n <= 0) return CBIS_OK;
  const size_t total = (size_t)rows * n;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(blend_rows_kernel<float>, dim3((int)blocks), dim3(256), 0, st, (const float*)a, a_ld,
                           (const float*)b, b_ld, (float*)out, out_ld, lambda, rows, n);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(blend_rows_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, st,
                           (const __nv_bfloat16*)a, a_ld, (const __nv_bfloat16*)b, b_ld, (__nv_bfloat16*)out, out_ld,
                           lambda, rows, n);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_rope_rows(const void* src, int src_ld, int src_col0, int src_head_stride, void* dst, int dst_ld,
                               int dst_col0, int dst_head_stride, const int* positions, int rows, int heads, int width,
                               int dims, const float* freqs, int dtype, void* stream, int neighbours, float length,
                               int keep, int keep_head0) {
  if (rows <= 0 || heads <= 0 || width <= 0) return CBIS_OK;
  if (dims < 0 || dims > width || dims % 2 || (dims > 0 && !freqs)) return CBIS_ERR_BAD_SIZE;
  const int units = heads * (dims / 2 + width - dims);
  const int threads = units >= 256 ? 256 : (units >= 128 ? 128 : 64);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(rope_rows_kernel<float>, dim3(rows), dim3(threads), 0, st, (const float*)src, src_ld, src_col0,
                           src_head_stride, (float*)dst, dst_ld, dst_col0, dst_head_stride, positions, heads, width, dims,
                           freqs, neighbours, length, keep, keep_head0);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(rope_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, st, (const __nv_bfloat16*)src,
                           src_ld, src_col0, src_head_stride, (__nv_bfloat16*)dst, dst_ld, dst_col0, dst_head_stride,
                           positions, heads, width, dims, freqs, neighbours, length, keep, keep_head0);
  return CBIS_ERR_BAD_DTYPE;
}

// gate_dtype: the gate's numbers may be 32-bit beside values of the compute type.
CBIS_EXPORT int cbis_head_gate_mul(const void* x, int x_ld, const void* gate, int gate_ld, int gate_dtype, void* out,
                                   int out_ld, int rows, int heads, int width, int dtype, void* stream) {
  if (rows <= 0 || heads <= 0 || width <= 0) return CBIS_OK;
  const size_t total = (size_t)rows * heads * width;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
#define CBIS_HG(TT, TG)                                                                                            \
  return (int)launch_pdl(head_gate_mul_kernel<TT, TG>, dim3((int)blocks), dim3(256), 0, st, (const TT*)x, x_ld,    \
                         (const TG*)gate, gate_ld, (TT*)out, out_ld, rows, heads, width)
  if (dtype == CBIS_F32 && gate_dtype == CBIS_F32) CBIS_HG(float, float);
  if (dtype == CBIS_BF16 && gate_dtype == CBIS_BF16) CBIS_HG(__nv_bfloat16, __nv_bfloat16);
  if (dtype == CBIS_BF16 && gate_dtype == CBIS_F32) CBIS_HG(__nv_bfloat16, float);
#undef CBIS_HG
  return CBIS_ERR_BAD_DTYPE;
}
