// Two small norms behind the recurrent mixers, float32 throughout, one rounding at the store:
//   group_rmsnorm_gate   out = o / sqrt(mean_group(o^2) + eps) * w * sigmoid(gate)      per group of n values of a row
//                        (a group = a head's values with one shared weight [n], or the whole row with a weight [G n])
//   rms_mean             x += (1 / B) * sum_b  y_b / sqrt(mean(y_b^2) + eps) * w_b        B <= 4 branches of one width
//   scale_add_group_rmsnorm   x <- N(alpha x + y), N the norm in groups with weight w [G n]; also h = x in another dtype
//                        (the norm behind a sublayer's sum: the stream, the sum and the norm in one pass)
#include "common.cuh"

namespace {
// A warp a (row, group) of at most 1,024 values (32 a lane, kept in registers between the two passes).
template <typename TH>
__global__ void __launch_bounds__(128)
k_scale_add_group_rmsnorm(float* __restrict__ x, const float* __restrict__ y, float alpha, const float* __restrict__ w,
                          TH* __restrict__ h, long long units, int groups, int n, float eps) {
  cima_pdl_wait();
  cima_pdl_trigger();
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const int grp = (int)(unit % groups);
  const size_t base = (size_t)unit * n;
  // Every load is issued without a condition (an index beyond the group reads the group's last value, which is then not
  // used), so that all of a lane's loads are in flight together: behind a branch each would wait for the one before it.
  float v[32], wv[32];
  const float* wp = w + (size_t)grp * n;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const int i = min(lane + 32 * j, n - 1);
    v[j] = x[base + i];
    wv[j] = wp[i];
  }
  if (y) {
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = fmaf(alpha, v[j], y[base + min(lane + 32 * j, n - 1)]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = alpha * v[j];
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    if (lane + 32 * j >= n) v[j] = 0.f;
    ss = fmaf(v[j], v[j], ss);
  }
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float r = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const int i = lane + 32 * j;
    if (i < n) {
      const float o = v[j] * r * wv[j];
      x[base + i] = o;
      if (h) h[base + i] = cima_from_f32<TH>(o);
    }
  }
}

// Longer groups: a block a (row, group), the sum read twice.
template <typename TH>
__global__ void __launch_bounds__(256)
k_scale_add_group_rmsnorm_wide(float* __restrict__ x, const float* __restrict__ y, float alpha, const float* __restrict__ w,
                               TH* __restrict__ h, int groups, int n, float eps) {
  cima_pdl_wait();
  cima_pdl_trigger();
  __shared__ float red[32];
  const long long unit = blockIdx.x;
  const int grp = (int)(unit % groups);
  const size_t base = (size_t)unit * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = y ? fmaf(alpha, x[base + i], y[base + i]) : alpha * x[base + i];
    ss = fmaf(v, v, ss);
  }
  ss = cima_block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)n + eps);
  const float* wp = w + (size_t)grp * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = y ? fmaf(alpha, x[base + i], y[base + i]) : alpha * x[base + i];
    const float o = v * r * wp[i];
    x[base + i] = o;
    if (h) h[base + i] = cima_from_f32<TH>(o);
  }
}

template <typename TH>
__global__ void __launch_bounds__(256)
k_cast_rows(const float* __restrict__ x, TH* __restrict__ h, size_t total) {
  cima_pdl_wait();
  cima_pdl_trigger();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;      // four values a thread
  if (i + 4 <= total && (((uintptr_t)x | (uintptr_t)h) & 15) == 0) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    if constexpr (sizeof(TH) == 2) {
      uint2 t;
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&t);
      h2[0] = __floats2bfloat162_rn(v.x, v.y);
      h2[1] = __floats2bfloat162_rn(v.z, v.w);
      *reinterpret_cast<uint2*>(h + i) = t;
    } else {
      *reinterpret_cast<float4*>(h + i) = v;
    }
    return;
  }
  for (size_t j = i; j < total && j < i + 4; j++) h[j] = cima_from_f32<TH>(x[j]);
}

template <typename TG, typename TO>
__global__ void __launch_bounds__(128)
k_group_rmsnorm_gate(const float* __restrict__ o, const float* __restrict__ w, const TG* __restrict__ gate, int ldg,
                     TO* __restrict__ out, long long units, int groups, int n, int shared_w, float eps) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const long long row = unit / groups;
  const int grp = (int)(unit - row * groups);
  const float* src = o + ((size_t)row * groups + grp) * n;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) ss = fmaf(src[i], src[i], ss);
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float r = 1.0f / sqrtf(ss / (float)n + eps);
  const float* wp = w + (shared_w ? 0 : (size_t)grp * n);
  const TG* gp = gate ? gate + (size_t)row * ldg + (size_t)grp * n : nullptr;
  TO* dst = out + ((size_t)row * groups + grp) * n;
  for (int i = lane; i < n; i += 32) {
    float y = src[i] * r * wp[i];
    if (gp) y *= 1.0f / (1.0f + expf(-cima_to_f32<TG>(gp[i])));
    dst[i] = cima_from_f32<TO>(y);
  }
}

// The same for long groups (a whole row of some thousand values): a block a (row, group).
template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
k_group_rmsnorm_gate_wide(const float* __restrict__ o, const float* __restrict__ w, const TG* __restrict__ gate, int ldg,
                          TO* __restrict__ out, int groups, int n, int shared_w, float eps) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  __shared__ float red[32];
  const long long unit = blockIdx.x;
  const long long row = unit / groups;
  const int grp = (int)(unit - row * groups);
  const float* src = o + ((size_t)row * groups + grp) * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
  ss = cima_block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)n + eps);
  const float* wp = w + (shared_w ? 0 : (size_t)grp * n);
  const TG* gp = gate ? gate + (size_t)row * ldg + (size_t)grp * n : nullptr;
  TO* dst = out + ((size_t)row * groups + grp) * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float y = src[i] * r * wp[i];
    if (gp) y *= 1.0f / (1.0f + expf(-cima_to_f32<TG>(gp[i])));
    dst[i] = cima_from_f32<TO>(y);
  }
}

struct Branches { const float* y[4]; const float* w[4]; int n; };

__global__ void __launch_bounds__(256)
k_rms_mean(Branches br, float* __restrict__ x, int H, float eps, int assign) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  float r[4];
  for (int b = 0; b < br.n; b++) {
    const float* y = br.y[b] + row * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) ss = fmaf(y[c], y[c], ss);
    ss = cima_block_sum(ss, red);
    r[b] = 1.0f / sqrtf(ss / (float)H + eps);
  }
  const float inv = 1.0f / (float)br.n;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < br.n; b++) s += br.y[b][row * H + c] * r[b] * br.w[b][c];
    x[row * H + c] = assign ? s * inv : x[row * H + c] + s * inv;
  }
}
}  // namespace

// o [T, groups * n] float32; w [n] (shared_w) or [groups * n]; gate [T, ldg] (gdtype) or null; out [T, groups * n] (odtype).
extern "C" int cima_group_rmsnorm_gate(const float* o, const float* w, const void* gate, int ldg, void* out, int dtype, int T,
                                       int groups, int n, int shared_w, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (groups <= 0 || n <= 0) return cima_fail(CIMA_E_SIZE, "group_rmsnorm_gate: %d groups of %d values must be positive", groups, n);
  const long long units = (long long)T * groups;
  const dim3 grid((unsigned)((units + 3) / 4));
  int rc;
  if (n >= 512 && units < 0x7fffffffll) {
    if (dtype == CIMA_F32) rc = cima_launch(k_group_rmsnorm_gate_wide<float, float>, dim3((unsigned)units), dim3(256), (size_t)0, stream, 1, o, w, (const float*)gate, ldg, (float*)out, groups, n, shared_w, eps);
    else if (dtype == CIMA_BF16) rc = cima_launch(k_group_rmsnorm_gate_wide<__nv_bfloat16, __nv_bfloat16>, dim3((unsigned)units), dim3(256), (size_t)0, stream, 1, o, w, (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)out, groups, n, shared_w, eps);
    else return cima_fail(CIMA_E_DTYPE, "group_rmsnorm_gate: dtype code %d is neither float32 nor bfloat16", dtype);
    return rc ? rc : cima_launch_result();
  }
  if (dtype == CIMA_F32) rc = cima_launch(k_group_rmsnorm_gate<float, float>, grid, dim3(128), (size_t)0, stream, 1, o, w, (const float*)gate, ldg, (float*)out, units, groups, n, shared_w, eps);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_group_rmsnorm_gate<__nv_bfloat16, __nv_bfloat16>, grid, dim3(128), (size_t)0, stream, 1, o, w, (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)out, units, groups, n, shared_w, eps);
  else return cima_fail(CIMA_E_DTYPE, "group_rmsnorm_gate: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}

// ys / ws: n_branches pointers to float32 [T, H] and [H]; x [T, H] float32 is added to, or with assign != 0 written.
extern "C" int cima_rms_mean(const float* const* ys, const float* const* ws, int n_branches, float* x, int T, int H, float eps,
                             int assign, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_branches < 1 || n_branches > 4 || H <= 0) return cima_fail(CIMA_E_SIZE, "rms_mean: %d branches (1..4) of width %d", n_branches, H);
  Branches br{};
  br.n = n_branches;
  for (int b = 0; b < n_branches; b++) { br.y[b] = ys[b]; br.w[b] = ws[b]; }
  int rc = cima_launch(k_rms_mean, dim3(T), dim3(256), (size_t)0, stream, 1, br, x, H, eps, assign);
  return rc ? rc : cima_launch_result();
}

// x [T, groups * n] float32 becomes N(alpha x + y) (y float32 of the same shape, or null for N(alpha x)); w [groups * n];
// h (hdtype, may be null) receives the same rows in that dtype.
extern "C" int cima_scale_add_group_rmsnorm(float* x, const float* y, float alpha, const float* w, void* h, int hdtype, int T,
                                            int groups, int n, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (groups <= 0 || n <= 0) return cima_fail(CIMA_E_SIZE, "scale_add_group_rmsnorm: %d groups of %d values must be positive", groups, n);
  if (h && hdtype != CIMA_F32 && hdtype != CIMA_BF16) return cima_fail(CIMA_E_DTYPE, "scale_add_group_rmsnorm: dtype code %d is neither float32 nor bfloat16", hdtype);
  const long long units = (long long)T * groups;
  if (units >= 0x7fffffffll) return cima_fail(CIMA_E_SIZE, "scale_add_group_rmsnorm: %d rows x %d groups exceed one launch", T, groups);
  int rc;
  if (n <= 1024) {
    const dim3 grid((unsigned)((units + 3) / 4));
    if (h && hdtype == CIMA_BF16) rc = cima_launch(k_scale_add_group_rmsnorm<__nv_bfloat16>, grid, dim3(128), (size_t)0, stream, 1, x, y, alpha, w, (__nv_bfloat16*)h, units, groups, n, eps);
    else rc = cima_launch(k_scale_add_group_rmsnorm<float>, grid, dim3(128), (size_t)0, stream, 1, x, y, alpha, w, (float*)h, units, groups, n, eps);
  } else {
    if (h && hdtype == CIMA_BF16) rc = cima_launch(k_scale_add_group_rmsnorm_wide<__nv_bfloat16>, dim3((unsigned)units), dim3(256), (size_t)0, stream, 1, x, y, alpha, w, (__nv_bfloat16*)h, groups, n, eps);
    else rc = cima_launch(k_scale_add_group_rmsnorm_wide<float>, dim3((unsigned)units), dim3(256), (size_t)0, stream, 1, x, y, alpha, w, (float*)h, groups, n, eps);
  }
  return rc ? rc : cima_launch_result();
}

// h = x in another dtype (the rows a sublayer reads where no norm stands in front of it).
extern "C" int cima_cast_rows(const float* x, void* h, int hdtype, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const size_t blocks = (total + 1023) / 1024;
  if (blocks > 0x7fffffffull) return cima_fail(CIMA_E_SIZE, "cast_rows: %zu values exceed one launch", total);
  int rc;
  if (hdtype == CIMA_BF16) rc = cima_launch(k_cast_rows<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), (size_t)0, stream, 1, x, (__nv_bfloat16*)h, total);
  else if (hdtype == CIMA_F32) rc = cima_launch(k_cast_rows<float>, dim3((unsigned)blocks), dim3(256), (size_t)0, stream, 1, x, (float*)h, total);
  else return cima_fail(CIMA_E_DTYPE, "cast_rows: dtype code %d is neither float32 nor bfloat16", hdtype);
  return rc ? rc : cima_launch_result();
}
