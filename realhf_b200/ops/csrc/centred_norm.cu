// Bias-free LayerNorm of "layer" stacks, fused with the residual add around it (fp32 arithmetic whatever the storage types; a
// type code per tensor; compiled without fast-math):
//
//   LN(v) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w          (the variance from the squared deviations: two passes
//                                                                           over the row, which sits in shared memory)
//   branch = a * y + b * y2                                                 (y2 optional: two mixers that ran side by side)
//   res   += mult * scale * LN_post(branch)                                 (res optional; scale optional)
//   out    = LN_next(res)            or, without res,   out = LN_next(branch)
//
// One CTA per row; every reduction runs over a fixed thread-to-element map and a fixed tree, so a row's result does not depend on
// the batch it is in.  Rows of a multiple of 4 elements with 16-byte aligned tensors take 16-byte / 8-byte accesses.
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

constexpr int kThreads = 256;

struct NormParams {
  void* res; int dtr;                 // [T, W] updated in place, or null
  const void* y; int64_t ldy; int dty;
  const void* y2; int64_t ldy2;       // same type as y, or null
  float a, b;
  const void* w_post;                 // [W] or null (with res: required)
  const void* scale;                  // [W] or null
  const void* w_next;                 // [W] or null
  int dtw;                            // type of the three weight vectors
  float mult;
  void* out; int dto;                 // [T, W] or null
  int W; float eps;
};

// mean and reciprocal standard deviation of row[0 .. W) in shared memory
RB_DEVICE void row_stats(const float* row, int W, float eps, float* red, float& mean, float& rstd) {
  float s = 0.f;
  for (int e = threadIdx.x; e < W; e += kThreads) s += row[e];
  mean = rb::block_reduce<false>(s, red) / (float)W;
  float ss = 0.f;
  for (int e = threadIdx.x; e < W; e += kThreads) { const float d = row[e] - mean; ss = fmaf(d, d, ss); }
  rstd = 1.f / sqrtf(rb::block_reduce<false>(ss, red) / (float)W + eps);
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads) centred_norm_kernel(NormParams p) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int W = p.W;
  rb::pdl_trigger();
  rb::pdl_wait();
  if constexpr (kVec) {
    for (int e = threadIdx.x * 4; e < W; e += kThreads * 4) {
      float4 v = rb::ld4_any(p.y, p.dty, t * p.ldy + e);
      v = make_float4(v.x * p.a, v.y * p.a, v.z * p.a, v.w * p.a);
      if (p.y2 != nullptr) {
        const float4 u = rb::ld4_any(p.y2, p.dty, t * p.ldy2 + e);
        v = make_float4(fmaf(u.x, p.b, v.x), fmaf(u.y, p.b, v.y), fmaf(u.z, p.b, v.z), fmaf(u.w, p.b, v.w));
      }
      *reinterpret_cast<float4*>(row + e) = v;
    }
  } else {
    for (int e = threadIdx.x; e < W; e += kThreads) {
      float v = ld_any(p.y, p.dty, t * p.ldy + e) * p.a;
      if (p.y2 != nullptr) v = fmaf(ld_any(p.y2, p.dty, t * p.ldy2 + e), p.b, v);
      row[e] = v;
    }
  }
  __syncthreads();
  float mean, rstd;
  if (p.res != nullptr) {
    row_stats(row, W, p.eps, red, mean, rstd);
    // every thread rewrites only the elements it owns below, so no barrier is needed between the statistics and the update
    for (int e = threadIdx.x; e < W; e += kThreads) {
      float n = (row[e] - mean) * rstd * ld_any(p.w_post, p.dtw, e);
      if (p.scale != nullptr) n *= ld_any(p.scale, p.dtw, e);
      const float r = ld_any(p.res, p.dtr, t * (int64_t)W + e) + p.mult * n;
      st_any(p.res, p.dtr, t * (int64_t)W + e, r);
      row[e] = rb::round_any(p.dtr, r);
    }
    if (p.out == nullptr) return;
    __syncthreads();
  }
  row_stats(row, W, p.eps, red, mean, rstd);
  if constexpr (kVec) {
    for (int e = threadIdx.x * 4; e < W; e += kThreads * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + e), w = rb::ld4_any(p.w_next, p.dtw, e);
      rb::st4_any(p.out, p.dto, t * (int64_t)W + e,
                  make_float4((v.x - mean) * rstd * w.x, (v.y - mean) * rstd * w.y, (v.z - mean) * rstd * w.z, (v.w - mean) * rstd * w.w));
    }
  } else {
    for (int e = threadIdx.x; e < W; e += kThreads) st_any(p.out, p.dto, t * (int64_t)W + e, (row[e] - mean) * rstd * ld_any(p.w_next, p.dtw, e));
  }
}

inline bool al16(const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

}  // namespace

// res [T, W] (type dtr) or null; y / y2 rows of stride ldy / ldy2 (type dty); the weight vectors share type dtw; out [T, W] (dto).
extern "C" int rb_centred_norm(void* res, int dtr, const void* y, int64_t ldy, const void* y2, int64_t ldy2, int dty, float a, float b,
                               const void* w_post, const void* scale, const void* w_next, int dtw, float mult, void* out, int dto, int64_t T,
                               int W, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (W < 1 || (res != nullptr && w_post == nullptr) || ((out == nullptr) != (w_next == nullptr)) || (res == nullptr && out == nullptr)) return -1;
  const size_t smem = (size_t)W * sizeof(float);
  if (smem > 160 * 1024) return -1;
  NormParams p{res, dtr, y, ldy, dty, y2, ldy2, a, b, w_post, scale, w_next, dtw, mult, out, dto, W, eps};
  const bool vec = W % 4 == 0 && ldy % 4 == 0 && (y2 == nullptr || ldy2 % 4 == 0) && al16(y) && al16(y2) && al16(w_next) && al16(out);
  auto kern = vec ? centred_norm_kernel<true> : centred_norm_kernel<false>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  return rb::launch_pdl(kern, dim3((unsigned)T), dim3(kThreads), smem, s, p) == cudaSuccess ? 0 : 2;
}
