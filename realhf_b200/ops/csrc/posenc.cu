// Small row-wise kernels of heterogeneous stacks that must keep exact libm functions (compiled without fast-math):
//   embed_sinusoid   x[t] = wte[ids[t]] + pe(p_t) in fp32; pe[2i] = sin(p f_i), pe[2i + 1] = cos(p f_i), the angle p * f_i formed
//                    in fp32 from the fp32 table f (rounded once from float64 on the host)
//   concat_cast      [a | b] along the last dim into one tensor of another type (the input of a projection reading two streams)
//   relu2            relu(x)^2
//   rms_norm_rows    out = x / sqrt(mean(x^2) + eps) * (w + w_off) per row (fp32 statistics, any storage types); with a branch output y it
//                    first forms x <- x + y in place (fp32 sum stored in x's type): the residual add fused into the next norm
#include "anytype.cuh"

namespace {

__global__ void embed_sinusoid_kernel(const int64_t* __restrict__ ids, const void* __restrict__ wte, int dtw, const int* __restrict__ pos,
                                      const int* __restrict__ slots, const float* __restrict__ inv_freq, float* __restrict__ out, int W, int vocab) {
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  int64_t id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float p = (float)(slots ? pos[slots[t]] : pos[t]);
  for (int i = threadIdx.x; i < W / 2; i += blockDim.x) {
    const float ang = p * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    out[t * W + 2 * i] = rb::ld_any(wte, dtw, id * W + 2 * i) + s;
    out[t * W + 2 * i + 1] = rb::ld_any(wte, dtw, id * W + 2 * i + 1) + c;
  }
  if ((W & 1) && threadIdx.x == 0) {  // odd width: the last column has no cosine partner
    const float ang = p * inv_freq[W / 2];
    out[t * W + W - 1] = rb::ld_any(wte, dtw, id * W + W - 1) + sinf(ang);
  }
}

__global__ void concat_cast_kernel(const void* __restrict__ a, int dta, int Wa, const void* __restrict__ b, int dtb, int Wb, void* __restrict__ out,
                                   int dto) {
  const int64_t t = blockIdx.x;
  const int W = Wa + Wb;
  rb::pdl_trigger();
  rb::pdl_wait();
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = i < Wa ? rb::ld_any(a, dta, t * Wa + i) : rb::ld_any(b, dtb, t * Wb + (i - Wa));
    rb::st_any(out, dto, t * W + i, v);
  }
}

__global__ void relu2_kernel(const void* __restrict__ x, void* __restrict__ out, int dt, int64_t n) {
  const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  rb::pdl_trigger();
  rb::pdl_wait();
  if (i0 + 3 < n) {
    float4 v = rb::ld4_any(x, dt, i0);
    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
    rb::st4_any(out, dt, i0, make_float4(v.x * v.x, v.y * v.y, v.z * v.z, v.w * v.w));
  } else {
    for (int64_t i = i0; i < n; ++i) { const float v = fmaxf(rb::ld_any(x, dt, i), 0.f); rb::st_any(out, dt, i, v * v); }
  }
}

// one CTA per row; the row is read once from DRAM (second pass from L1 / L2)
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(void* __restrict__ x, int dtx, const void* __restrict__ y, int dty,
                                                            const void* __restrict__ w, int dtw, void* __restrict__ out, int dto, int W, float eps,
                                                            float w_off) {
  __shared__ float red[32];
  const int64_t base = (int64_t)blockIdx.x * W;
  const bool vec = (W & 3) == 0;
  float ss = 0.f;
  rb::pdl_trigger();
  rb::pdl_wait();
  if (vec) {
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      float4 v = rb::ld4_any(x, dtx, base + i);
      if (y != nullptr) {
        const float4 b = rb::ld4_any(y, dty, base + i);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        rb::st4_any(x, dtx, base + i, v);
        if (dtx != 0) v = make_float4(rb::round_any(dtx, v.x), rb::round_any(dtx, v.y), rb::round_any(dtx, v.z), rb::round_any(dtx, v.w));
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = rb::ld_any(x, dtx, base + i);
      if (y != nullptr) { v += rb::ld_any(y, dty, base + i); rb::st_any(x, dtx, base + i, v); v = rb::round_any(dtx, v); }
      ss += v * v;
    }
  }
  ss = rb::block_reduce<false>(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  // every thread re-reads exactly the elements it wrote above, so no barrier is needed for the in-place sum
  if (vec) {
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      const float4 v = rb::ld4_any(x, dtx, base + i), g = rb::ld4_any(w, dtw, i);
      rb::st4_any(out, dto, base + i, make_float4(v.x * r * (g.x + w_off), v.y * r * (g.y + w_off), v.z * r * (g.z + w_off), v.w * r * (g.w + w_off)));
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) rb::st_any(out, dto, base + i, rb::ld_any(x, dtx, base + i) * r * (rb::ld_any(w, dtw, i) + w_off));
  }
}

}  // namespace

extern "C" int rb_rms_norm_rows(void* x, int dtx, const void* y, int dty, const void* w, int dtw, void* out, int dto, int64_t rows, int W, float eps,
                                float w_off, cudaStream_t s) {
  if (rows == 0) return 0;
  return rb::launch_pdl(rms_norm_rows_kernel, dim3((unsigned)rows), dim3(256), 0, s, x, dtx, y, dty, w, dtw, out, dto, W, eps, w_off) == cudaSuccess ? 0 : -3;
}

extern "C" int rb_embed_sinusoid(const int64_t* ids, const void* wte, int dtw, const int* pos, const int* slots, const float* inv_freq, float* out,
                                 int64_t T, int W, int vocab, cudaStream_t s) {
  if (T == 0) return 0;
  return rb::launch_pdl(embed_sinusoid_kernel, dim3((unsigned)T), dim3(128), 0, s, ids, wte, dtw, pos, slots, inv_freq, out, W, vocab) == cudaSuccess ? 0 : -3;
}

extern "C" int rb_concat_cast(const void* a, int dta, int Wa, const void* b, int dtb, int Wb, void* out, int dto, int64_t T, cudaStream_t s) {
  if (T == 0) return 0;
  return rb::launch_pdl(concat_cast_kernel, dim3((unsigned)T), dim3(256), 0, s, a, dta, Wa, b, dtb, Wb, out, dto) == cudaSuccess ? 0 : -3;
}

extern "C" int rb_relu2(const void* x, void* out, int dt, int64_t n, cudaStream_t s) {
  if (n == 0) return 0;
  const int64_t blocks = (n + 1023) / 1024;
  return rb::launch_pdl(relu2_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, out, dt, n) == cudaSuccess ? 0 : -3;
}
