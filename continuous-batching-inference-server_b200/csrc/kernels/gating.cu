// Gates and unit norms, all in 32-bit arithmetic whatever the storage type:
//   * rms_norm: rows divided by their root mean square in equal parts, times a weight; an optional gate
//     (act(z), element by element) is applied BEFORE the norm, or (gate_after) to the normalised, weighted values;
//   * gate_mul: out = act(a) * b, the inside of a gated feed-forward (a = gate, b = up) and an output gate
//     (a = the gate's projection, b = the values, act = sigmoid).
#include "common.cuh"

namespace cbis {

// grid (rows, parts); part g of row r covers columns g*pw .. g*pw + pw - 1.
//   v = x[r, c] * (gate ? act(gate[r, c]) : 1);  out[r, c] = v / sqrt(mean_c(v^2) + eps) * (weight ? weight[c] : 1)
// With gate_after the gate stays out of v:  out[r, c] = x / sqrt(mean_c(x^2) + eps) * weight[c] * act(gate[r, c]).
// With `staged` the part's v wait in shared memory (pw floats) between the two passes; else they are read again.
template <typename TI, typename TG, typename TO>
__global__ void rms_norm_kernel(const TI* x, int x_ld, const TG* gate, int gate_ld, int gate_act,
                                const float* __restrict__ weight, float eps, TO* out, int out_ld, int pw, int staged,
                                int gate_after) {
  extern __shared__ float vs[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, c0 = blockIdx.y * pw;
  const TI* xr = x + (size_t)r * x_ld + c0;
  const TG* gr = gate ? gate + (size_t)r * gate_ld + c0 : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < pw; c += blockDim.x) {
    float v = to_f32(xr[c]);
    if (gr && !gate_after) v *= activate(to_f32(gr[c]), gate_act);
    if (staged) vs[c] = v;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)pw + eps);
  TO* orow = out + (size_t)r * out_ld + c0;
  for (int c = threadIdx.x; c < pw; c += blockDim.x) {
    float v;
    if (staged) {
      v = vs[c];
    } else {
      v = to_f32(xr[c]);
      if (gr && !gate_after) v *= activate(to_f32(gr[c]), gate_act);
    }
    v *= inv;
    if (weight) v *= weight[c0 + c];
    if (gr && gate_after) v *= activate(to_f32(gr[c]), gate_act);
    from_f32(orow[c], v);
  }
}

// out[r, c] = act(a[r, c]) * b[r, c]; with `b_rows` b's row is b_rows[r] instead (rows of a table looked up by token;
// an index outside 0 .. b_n_rows - 1 reads as zeros)
template <typename TT>
__global__ void gate_mul_kernel(const TT* a, int a_ld, const TT* b, int b_ld, TT* out, int out_ld, int act, int rows,
                                int n, const int* b_rows, int b_n_rows) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n;
    const int c = (int)(i % n);
    size_t br = r;
    bool there = true;
    if (b_rows) {
      const int t = b_rows[r];
      there = t >= 0 && t < b_n_rows;
      br = there ? (size_t)t : 0;
    }
    const float bv = there ? to_f32(b[br * b_ld + c]) : 0.f;
    from_f32(out[r * out_ld + c], activate(to_f32(a[r * a_ld + c]), act) * bv);
  }
}

template <typename TI, typename TG, typename TO>
static int launch_rms(const void* x, int x_ld, const void* gate, int gate_ld, int gate_act, const float* weight,
                      float eps, void* out, int out_ld, int rows, int parts, int pw, int gate_after, cudaStream_t st) {
  const int threads = pw >= 2048 ? 512 : (pw >= 512 ? 256 : (pw >= 128 ? 128 : 64));
  const int staged = pw <= 10240 ? 1 : 0;         // 40 KB of shared memory at most
  return (int)launch_pdl(rms_norm_kernel<TI, TG, TO>, dim3(rows, parts), dim3(threads),
                         staged ? (size_t)pw * sizeof(float) : 0, st, (const TI*)x, x_ld, (const TG*)gate, gate_ld,
                         gate_act, weight, eps, (TO*)out, out_ld, pw, staged, gate_after);
}

}  // namespace cbis

using namespace cbis;

// x: 32-bit or the compute type (x_dtype); gate (may be null) and out: the compute type (dtype).
CBIS_EXPORT int cbis_rms_norm(const void* x, int x_ld, int x_dtype, const void* gate, int gate_ld, int gate_act,
                              const float* weight, float eps, void* out, int out_ld, int dtype, int rows, int parts,
                              int part_width, void* stream, int gate_after) {
  if (rows <= 0) return CBIS_OK;
  if (parts <= 0 || part_width <= 0) return CBIS_ERR_BAD_SIZE;
  if (parts > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
#define CBIS_RMS(TI, TG) \
  return launch_rms<TI, TG, TG>(x, x_ld, gate, gate_ld, gate_act, weight, eps, out, out_ld, rows, parts, part_width, gate_after, st)
  if (dtype == CBIS_F32 && x_dtype == CBIS_F32) CBIS_RMS(float, float);
  if (dtype == CBIS_BF16 && x_dtype == CBIS_F32) CBIS_RMS(float, __nv_bfloat16);
  if (dtype == CBIS_BF16 && x_dtype == CBIS_BF16) CBIS_RMS(__nv_bfloat16, __nv_bfloat16);
#undef CBIS_RMS
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_gate_mul(const void* a, int a_ld, const void* b, int b_ld, void* out, int out_ld, int act, int rows,
                              int n, int dtype, void* stream, const int* b_rows, int b_n_rows) {
  if (rows <= 0 || n <= 0) return CBIS_OK;
  const size_t total = (size_t)rows * n;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(gate_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, st, (const float*)a, a_ld,
                           (const float*)b, b_ld, (float*)out, out_ld, act, rows, n, b_rows, b_n_rows);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(gate_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, st, (const __nv_bfloat16*)a,
                           a_ld, (const __nv_bfloat16*)b, b_ld, (__nv_bfloat16*)out, out_ld, act, rows, n, b_rows, b_n_rows);
  return CBIS_ERR_BAD_DTYPE;
}
