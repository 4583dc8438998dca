// Several copies of the residual stream ("hyper-connections") and an ungated activation.
//
// hyper_connect: the streams X [T, S, W] float32 take a sublayer's output y [T, W] and are read for the next sublayer:
//   write   X_t <- sum_s C[s, t] X_s + mult * b[t] * y      for all t at once, from the old X   (C [S, S] indexed [from, to])
//           (spread: X_t <- y for all t: the copies start equal to the embedding's rows)
//   read    u = sum_s a[s] X_s (the new X);   h = u / sqrt(mean(u^2) + eps) * w                  (w: the norm's weight as applied)
// One block a row.  A thread owns the columns c = tid, tid + threads, ...: it loads the S old values of a column, forms the
// S new ones and the reader's sum in registers, stores the new values and keeps u (the first U_KEEP columns of a thread
// in registers, the rest are formed again from the streams it wrote itself).  The sum of squares is added in a fixed
// order (cima_block_sum), so a row's result does not depend on what else is in the launch.  Everything float32; h is
// rounded once at its store.  S <= 8.  Two forms: for up to four streams of a width that is a multiple of 4, a thread
// takes four neighbouring columns at a time (16-byte loads and stores) and requests everything it will read, for up to
// four such groups, before it computes: a decode step's few rows are one trip to memory deep, a prompt's rows keep the
// memory busy.  Any other size takes the form that walks column by column.
//
// activate: z <- act(z) in place for an ungated feed-forward's middle (the gate activations, and relu2 = relu(z)^2).
#include "common.cuh"

namespace {
constexpr int HC_MAX_STREAMS = 8;
constexpr int HC_THREADS = 256;
constexpr int U_KEEP = 8;             // columns of a thread whose sum stays in registers (W <= 2048 at 256 threads)

template <typename TH>
__global__ void __launch_bounds__(HC_THREADS)
k_hyper_connect(float* __restrict__ X, const float* __restrict__ y, const float* __restrict__ C, const float* __restrict__ b,
                float mult, int spread, const float* __restrict__ a, const float* __restrict__ w, float eps, TH* __restrict__ h,
                int S, int W) {
  __shared__ float red[32];
  __shared__ float sC[HC_MAX_STREAMS * HC_MAX_STREAMS], sb[HC_MAX_STREAMS], sa[HC_MAX_STREAMS];
  // the connection's numbers do not depend on the kernel before this one: they are fetched before the wait
  if (threadIdx.x < S * S && C) sC[threadIdx.x] = C[threadIdx.x];
  if (threadIdx.x < S) {
    if (b) sb[threadIdx.x] = mult * b[threadIdx.x];
    if (a) sa[threadIdx.x] = a[threadIdx.x];
  }
  cima_pdl_wait();
  __syncthreads();
  const size_t row = blockIdx.x;
  float* xr = X + row * (size_t)S * W;
  const float* yr = y ? y + row * (size_t)W : nullptr;
  float keep[U_KEEP];
  float ss = 0.f;
  int n = 0;
  for (int c = threadIdx.x; c < W; c += HC_THREADS, n++) {
    float nw[HC_MAX_STREAMS];
    if (yr && spread) {
      const float v = yr[c];
#pragma unroll
      for (int t = 0; t < HC_MAX_STREAMS; t++)
        if (t < S) { nw[t] = v; xr[(size_t)t * W + c] = v; }
    } else {
      float old[HC_MAX_STREAMS];
#pragma unroll
      for (int s = 0; s < HC_MAX_STREAMS; s++) old[s] = s < S ? xr[(size_t)s * W + c] : 0.f;
      if (yr) {
        const float v = yr[c];
#pragma unroll
        for (int t = 0; t < HC_MAX_STREAMS; t++) {
          if (t < S) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; s++)
              if (s < S) acc = fmaf(sC[s * S + t], old[s], acc);
            nw[t] = fmaf(sb[t], v, acc);
            xr[(size_t)t * W + c] = nw[t];
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < HC_MAX_STREAMS; t++) nw[t] = old[t];
      }
    }
    if (a) {
      float u = 0.f;
#pragma unroll
      for (int t = 0; t < HC_MAX_STREAMS; t++)
        if (t < S) u = fmaf(sa[t], nw[t], u);
      if (n < U_KEEP) keep[n] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!a) return;
  const float total = cima_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)W + eps);
  TH* hr = h + row * (size_t)W;
  n = 0;
  for (int c = threadIdx.x; c < W; c += HC_THREADS, n++) {
    float u;
    if (n < U_KEEP) {
      u = keep[n];
    } else {                              // formed again, in the same order, from what this thread stored
      u = 0.f;
#pragma unroll
      for (int t = 0; t < HC_MAX_STREAMS; t++)
        if (t < S) u = fmaf(sa[t], xr[(size_t)t * W + c], u);
    }
    hr[c] = cima_from_f32<TH>(u * inv * w[c]);
  }
}

__device__ __forceinline__ float4 f4_fma(float a, float4 x, float4 acc) {
  return make_float4(fmaf(a, x.x, acc.x), fmaf(a, x.y, acc.y), fmaf(a, x.z, acc.z), fmaf(a, x.w, acc.w));
}
template <typename TH> __device__ __forceinline__ void store4(TH* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 t;
  *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = t;
}

constexpr int HC_GROUPS = 4;          // groups of four columns a thread holds at a time (a pass covers 4,096 columns)

template <typename TH, int S>
__global__ void __launch_bounds__(HC_THREADS)
k_hyper_connect4(float* __restrict__ X, const float* __restrict__ y, const float* __restrict__ C, const float* __restrict__ b,
                 float mult, int spread, const float* __restrict__ a, const float* __restrict__ w, float eps, TH* __restrict__ h, int W) {
  __shared__ float red[32];
  float rC[S * S], rb[S], ra[S];
#pragma unroll
  for (int i = 0; i < S * S; i++) rC[i] = C ? C[i] : 0.f;
#pragma unroll
  for (int i = 0; i < S; i++) { rb[i] = b ? mult * b[i] : 0.f; ra[i] = a ? a[i] : 0.f; }
  const int W4 = W >> 2, NT = blockDim.x;       // 128 threads where they cover the row in four groups, else 256
  const size_t row = blockIdx.x;
  // the norm's weight does not depend on the kernel before this one either
  float4 wv[HC_GROUPS];
#pragma unroll
  for (int k = 0; k < HC_GROUPS; k++) {
    const int g = threadIdx.x + k * NT;
    wv[k] = (a && g < W4) ? reinterpret_cast<const float4*>(w)[g] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  cima_pdl_wait();
  float4* xr = reinterpret_cast<float4*>(X + row * (size_t)S * W);
  const float4* yr = y ? reinterpret_cast<const float4*>(y + row * (size_t)W) : nullptr;
  float4 keep[HC_GROUPS];
  float ss = 0.f;
  for (int g0 = 0; g0 < W4; g0 += HC_GROUPS * NT) {
    float4 old[HC_GROUPS][S], yv[HC_GROUPS];
#pragma unroll
    for (int k = 0; k < HC_GROUPS; k++) {                 // every load of the pass is requested here
      const int g = g0 + threadIdx.x + k * NT;
      const bool live = g < W4;
      yv[k] = (yr && live) ? yr[g] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s = 0; s < S; s++)
        old[k][s] = (live && !(yr && spread)) ? xr[(size_t)s * W4 + g] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < HC_GROUPS; k++) {
      const int g = g0 + threadIdx.x + k * NT;
      if (g >= W4) continue;
      float4 nw[S];
      if (yr && spread) {
#pragma unroll
        for (int t = 0; t < S; t++) { nw[t] = yv[k]; xr[(size_t)t * W4 + g] = nw[t]; }
      } else if (yr) {
#pragma unroll
        for (int t = 0; t < S; t++) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s = 0; s < S; s++) acc = f4_fma(rC[s * S + t], old[k][s], acc);
          nw[t] = f4_fma(rb[t], yv[k], acc);
          xr[(size_t)t * W4 + g] = nw[t];
        }
      } else {
#pragma unroll
        for (int t = 0; t < S; t++) nw[t] = old[k][t];
      }
      if (a) {
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int t = 0; t < S; t++) u = f4_fma(ra[t], nw[t], u);
        if (g0 == 0) keep[k] = u;
        ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
      }
    }
  }
  if (!a) return;
  const float total = cima_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)W + eps);
  TH* hr = h + row * (size_t)W;
#pragma unroll
  for (int k = 0; k < HC_GROUPS; k++) {
    const int g = threadIdx.x + k * NT;
    if (g >= W4) continue;
    const float4 u = keep[k];
    store4<TH>(hr + 4 * (size_t)g, make_float4(u.x * inv * wv[k].x, u.y * inv * wv[k].y, u.z * inv * wv[k].z, u.w * inv * wv[k].w));
  }
  for (int g = HC_GROUPS * NT + threadIdx.x; g < W4; g += NT) {      // beyond the first pass: formed again, in the same order
    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < S; t++) u = f4_fma(ra[t], xr[(size_t)t * W4 + g], u);
    const float4 ww = reinterpret_cast<const float4*>(w)[g];
    store4<TH>(hr + 4 * (size_t)g, make_float4(u.x * inv * ww.x, u.y * inv * ww.y, u.z * inv * ww.z, u.w * inv * ww.w));
  }
}

template <typename TH>
static int launch_hyper4(float* X, const float* y, const float* C, const float* b, float mult, int spread, const float* a, const float* w,
                         float eps, TH* h, int T, int S, int W, cudaStream_t stream) {
  const dim3 HC_BLOCK((W >> 2) <= HC_GROUPS * 128 ? 128 : HC_THREADS);      // every thread's groups are live where that covers the row
  switch (S) {
    case 1: return cima_launch(k_hyper_connect4<TH, 1>, dim3(T), HC_BLOCK, (size_t)0, stream, 1, X, y, C, b, mult, spread, a, w, eps, h, W);
    case 2: return cima_launch(k_hyper_connect4<TH, 2>, dim3(T), HC_BLOCK, (size_t)0, stream, 1, X, y, C, b, mult, spread, a, w, eps, h, W);
    case 3: return cima_launch(k_hyper_connect4<TH, 3>, dim3(T), HC_BLOCK, (size_t)0, stream, 1, X, y, C, b, mult, spread, a, w, eps, h, W);
    default: return cima_launch(k_hyper_connect4<TH, 4>, dim3(T), HC_BLOCK, (size_t)0, stream, 1, X, y, C, b, mult, spread, a, w, eps, h, W);
  }
}

__device__ __forceinline__ float ungated_act(float z, int act) {
  if (act == 5) { const float r = fmaxf(z, 0.f); return r * r; }
  return cima_gate_act(z, act);
}

template <typename TA>
__global__ void k_activate(TA* __restrict__ z, size_t total, int act) {
  cima_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    z[i] = cima_from_f32<TA>(ungated_act(cima_to_f32<TA>(z[i]), act));
}

__global__ void k_activate_bf16x8(__nv_bfloat16* __restrict__ z, size_t groups, int act) {
  cima_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
    uint4 v = *reinterpret_cast<const uint4*>(z + i * 8);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 f = __bfloat1622float2(p[e]);
      p[e] = __floats2bfloat162_rn(ungated_act(f.x, act), ungated_act(f.y, act));
    }
    *reinterpret_cast<uint4*>(z + i * 8) = v;
  }
}

}  // namespace

// X [T, S, W] float32 in place.  y (may be null) [T, W] float32 with C [S, S], b [S] (both null with spread != 0).
// a (may be null) [S] with w [W] and h [T, W] of h_dtype.
extern "C" int cima_hyper_connect(float* X, const float* y, const float* C, const float* b, float mult, int spread, const float* a,
                                  const float* w, float eps, void* h, int h_dtype, int T, int S, int W, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S < 1 || S > HC_MAX_STREAMS || W <= 0) return cima_fail(CIMA_E_SIZE, "hyper_connect: %d streams (1 to %d) of %d values", S, HC_MAX_STREAMS, W);
  if (y && !spread && (!C || !b)) return cima_fail(CIMA_E_ARG, "hyper_connect: writing a sublayer's output takes the matrix and the output vector");
  if (spread && !y) return cima_fail(CIMA_E_ARG, "hyper_connect: spreading takes the rows to spread");
  if (a && (!w || !h)) return cima_fail(CIMA_E_ARG, "hyper_connect: reading takes the norm's weight and a place for the rows");
  if (!y && !a) return 0;
  if (spread) { C = nullptr; b = nullptr; }
  int rc;
  if (a && h_dtype != CIMA_F32 && h_dtype != CIMA_BF16) return cima_fail(CIMA_E_DTYPE, "hyper_connect: dtype code %d is neither float32 nor bfloat16", h_dtype);
  if (S <= 4 && W % 4 == 0 && (((uintptr_t)X | (uintptr_t)y | (uintptr_t)w) & 15) == 0 && ((uintptr_t)h & 7) == 0) {
    if (!a || h_dtype == CIMA_F32) rc = launch_hyper4<float>(X, y, C, b, mult, spread, a, w, eps, (float*)h, T, S, W, stream);
    else rc = launch_hyper4<__nv_bfloat16>(X, y, C, b, mult, spread, a, w, eps, (__nv_bfloat16*)h, T, S, W, stream);
    return rc ? rc : cima_launch_result();
  }
  if (!a || h_dtype == CIMA_F32) rc = cima_launch(k_hyper_connect<float>, dim3(T), dim3(HC_THREADS), (size_t)0, stream, 1, X, y, C, b, mult, spread, a, w, eps, (float*)h, S, W);
  else if (h_dtype == CIMA_BF16) rc = cima_launch(k_hyper_connect<__nv_bfloat16>, dim3(T), dim3(HC_THREADS), (size_t)0, stream, 1, X, y, C, b, mult, spread, a, w, eps, (__nv_bfloat16*)h, S, W);
  else return cima_fail(CIMA_E_DTYPE, "hyper_connect: dtype code %d is neither float32 nor bfloat16", h_dtype);
  return rc ? rc : cima_launch_result();
}

extern "C" int cima_activate(void* z, int dtype, size_t total, int act, cudaStream_t stream) {
  if (total == 0) return 0;
  if (!((act >= 0 && act < CIMA_ACT_COUNT) || act == 5)) return cima_fail(CIMA_E_ARG, "activate: activation code %d is unknown", act);
  int rc;
  if (dtype == CIMA_BF16 && total % 8 == 0 && ((uintptr_t)z & 15) == 0) {
    const size_t groups = total / 8;
    const int grid = (int)((groups + 255) / 256 > 148 * 16 ? 148 * 16 : (groups + 255) / 256);
    rc = cima_launch(k_activate_bf16x8, dim3(grid), dim3(256), (size_t)0, stream, 1, (__nv_bfloat16*)z, groups, act);
    return rc ? rc : cima_launch_result();
  }
  const int grid = (int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
  if (dtype == CIMA_F32) rc = cima_launch(k_activate<float>, dim3(grid), dim3(256), (size_t)0, stream, 1, (float*)z, total, act);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_activate<__nv_bfloat16>, dim3(grid), dim3(256), (size_t)0, stream, 1, (__nv_bfloat16*)z, total, act);
  else return cima_fail(CIMA_E_DTYPE, "activate: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}
