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
// the batch it is in.  Rows of a multiple of 4 elements (up to 8192) with 16-byte aligned tensors keep the row in registers, four
// consecutive elements per 16-byte / 8-byte access: the residual row is fetched before the first reduction, and each norm takes two
// block reductions over the registers (the sum, then the squared deviations from the mean).  Other rows go through shared memory,
// element by element.
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

// ---- register form
// mean and reciprocal standard deviation of the row held as NV float4 per thread
template <int NV>
RB_DEVICE void reg_stats(const float4 (&v)[NV], int W, float eps, float* red, float& mean, float& rstd) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j)
    if ((threadIdx.x + j * kThreads) * 4 < W) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  mean = rb::block_reduce<false>(s, red) / (float)W;
  float m2 = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j)
    if ((threadIdx.x + j * kThreads) * 4 < W) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      m2 += (a * a + b * b) + (c * c + d * d);
    }
  rstd = 1.f / sqrtf(rb::block_reduce<false>(m2, red) / (float)W + eps);
}

// NV float4 per thread: rows of up to NV * 1024 elements
template <int NV>
__global__ void __launch_bounds__(kThreads) centred_norm_reg_kernel(NormParams p) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int W = p.W;
  rb::pdl_trigger();
  rb::pdl_wait();
  float4 v[NV], r[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int e = (threadIdx.x + j * kThreads) * 4;
    if (e < W) {
      v[j] = rb::ld4_any(p.y, p.dty, t * p.ldy + e);
      v[j] = make_float4(v[j].x * p.a, v[j].y * p.a, v[j].z * p.a, v[j].w * p.a);
      if (p.y2 != nullptr) {
        const float4 u = rb::ld4_any(p.y2, p.dty, t * p.ldy2 + e);
        v[j] = make_float4(fmaf(u.x, p.b, v[j].x), fmaf(u.y, p.b, v[j].y), fmaf(u.z, p.b, v[j].z), fmaf(u.w, p.b, v[j].w));
      }
      if (p.res != nullptr) r[j] = rb::ld4_any(p.res, p.dtr, t * (int64_t)W + e);
    }
  }
  if (p.res != nullptr) {
    float mean, rstd;
    reg_stats<NV>(v, W, p.eps, red, mean, rstd);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int e = (threadIdx.x + j * kThreads) * 4;
      if (e < W) {
        // the same products, in the same order, as the element-wise form: ((v - mean) rstd w_post) scale, times mult, plus res
        const float4 wp = rb::ld4_any(p.w_post, p.dtw, e);
        float4 n = make_float4((v[j].x - mean) * rstd * wp.x, (v[j].y - mean) * rstd * wp.y, (v[j].z - mean) * rstd * wp.z, (v[j].w - mean) * rstd * wp.w);
        if (p.scale != nullptr) { const float4 g = rb::ld4_any(p.scale, p.dtw, e); n = make_float4(n.x * g.x, n.y * g.y, n.z * g.z, n.w * g.w); }
        r[j] = make_float4(r[j].x + p.mult * n.x, r[j].y + p.mult * n.y, r[j].z + p.mult * n.z, r[j].w + p.mult * n.w);
        rb::st4_any(p.res, p.dtr, t * (int64_t)W + e, r[j]);
        v[j] = make_float4(rb::round_any(p.dtr, r[j].x), rb::round_any(p.dtr, r[j].y), rb::round_any(p.dtr, r[j].z), rb::round_any(p.dtr, r[j].w));
      }
    }
    if (p.out == nullptr) return;
  }
  float mean, rstd;
  reg_stats<NV>(v, W, p.eps, red, mean, rstd);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int e = (threadIdx.x + j * kThreads) * 4;
    if (e < W) {
      const float4 w = rb::ld4_any(p.w_next, p.dtw, e);
      rb::st4_any(p.out, p.dto, t * (int64_t)W + e,
                  make_float4((v[j].x - mean) * rstd * w.x, (v[j].y - mean) * rstd * w.y, (v[j].z - mean) * rstd * w.z, (v[j].w - mean) * rstd * w.w));
    }
  }
}

template <int NV>
int launch_reg(const NormParams& p, int64_t T, cudaStream_t s) {
  return rb::launch_pdl(centred_norm_reg_kernel<NV>, dim3((unsigned)T), dim3(kThreads), 0, s, p) == cudaSuccess ? 0 : 2;
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
  if (vec && W <= 8192 && al16(res) && al16(w_post) && al16(scale)) {
    if (W <= 1024) return launch_reg<1>(p, T, s);
    if (W <= 2048) return launch_reg<2>(p, T, s);
    if (W <= 4096) return launch_reg<4>(p, T, s);
    return launch_reg<8>(p, T, s);
  }
  auto kern = vec ? centred_norm_kernel<true> : centred_norm_kernel<false>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  return rb::launch_pdl(kern, dim3((unsigned)T), dim3(kThreads), smem, s, p) == cudaSuccess ? 0 : 2;
}
