// The end of a differential attention: two softmax maps over the same values are combined head by head,
//   o = a1 - lambda a2;   o <- o / sqrt(mean(o^2) + eps) * post;   o <- o * sigmoid(gate[head])
// with one lambda and one factor `post` for the layer and one gate value a head and row.  The maps come from an
// attention over 2 * heads query heads that stand in groups of `rep` heads sharing a key head: the block of 2 * rep
// heads of key-head pair g holds map 1 of the group's rep heads, then map 2 of the same heads, each `hd` values wide of
// which the first `vdim` count.  The output rows hold `heads * vdim` values, head by head in the model's order.
// Everything is float32; one rounding at the store.  A warp a (row, head).
#include "common.cuh"

namespace {
template <typename TA>
__global__ void __launch_bounds__(128)
k_diff_combine(const TA* __restrict__ att, int lda, const TA* __restrict__ gate, int ldg, TA* __restrict__ out, long long units,
               int heads, int rep, int hd, int vdim, float lambda, float post, float eps) {
  cima_pdl_wait();
  cima_pdl_trigger();        // a short kernel: the next one may be set up while this one runs (it waits for this one's end itself)
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const long long row = unit / heads;
  const int h = (int)(unit - row * heads);
  const int g = h / rep, i = h - g * rep;
  const TA* a1 = att + (size_t)row * lda + (size_t)(g * 2 * rep + i) * hd;
  const TA* a2 = a1 + (size_t)rep * hd;
  float o[8];                                                   // vdim <= 256: eight values a lane
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int d = lane + 32 * j;
    o[j] = d < vdim ? cima_to_f32<TA>(a1[d]) - lambda * cima_to_f32<TA>(a2[d]) : 0.f;
    ss = fmaf(o[j], o[j], ss);
  }
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  float r = post / sqrtf(ss / (float)vdim + eps);
  if (gate) r *= 1.0f / (1.0f + expf(-cima_to_f32<TA>(gate[(size_t)row * ldg + h])));
  TA* dst = out + ((size_t)row * heads + h) * vdim;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int d = lane + 32 * j;
    if (d < vdim) dst[d] = cima_from_f32<TA>(o[j] * r);
  }
}
}  // namespace

// att [T, lda]: 2 * heads heads of hd values (layout above); gate [T, ldg] with one value a head, or null; out [T, heads * vdim].
extern "C" int cima_diff_combine(const void* att, int lda, const void* gate, int ldg, void* out, int dtype, int T, int heads,
                                 int rep, int hd, int vdim, float lambda, float post, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || rep <= 0 || heads % rep) return cima_fail(CIMA_E_SIZE, "diff_combine: %d heads are not a multiple of the %d that share a key head", heads, rep);
  if (vdim <= 0 || vdim > hd || hd > 256) return cima_fail(CIMA_E_SIZE, "diff_combine: value size %d must lie in 1..head size %d <= 256", vdim, hd);
  if (lda < 2 * heads * hd) return cima_fail(CIMA_E_SIZE, "diff_combine: row stride %d is smaller than 2 * heads * head size = %d", lda, 2 * heads * hd);
  const long long units = (long long)T * heads;
  if ((units + 3) / 4 > 0x7fffffffll) return cima_fail(CIMA_E_SIZE, "diff_combine: %d rows x %d heads exceed one launch", T, heads);
  const dim3 grid((unsigned)((units + 3) / 4));
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_diff_combine<float>, grid, dim3(128), (size_t)0, stream, 1, (const float*)att, lda, (const float*)gate, ldg, (float*)out, units, heads, rep, hd, vdim, lambda, post, eps);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_diff_combine<__nv_bfloat16>, grid, dim3(128), (size_t)0, stream, 1, (const __nv_bfloat16*)att, lda, (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)out, units, heads, rep, hd, vdim, lambda, post, eps);
  else return cima_fail(CIMA_E_DTYPE, "diff_combine: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}
