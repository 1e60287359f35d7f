// Mixture-of-experts routing and combination for stacks that route by the softmax over all router outputs (fp32 arithmetic, any
// storage type; compiled without fast-math):
//   softmax_router   one CTA per token: logits z = W x (fp32 accumulation, the columns split over four warps), s = softmax(z) over
//                    all R outputs (or, `sigmoid`, s = 1 / (1 + exp(-z)) of every output on its own), the k largest of s + correction
//                    in descending order, their weights s (optionally divided by their sum); also, with an extra vector u, the
//                    token's gate sigmoid(u . x).  x is read once per 8 outputs (from L1 after the first pass).
//   moe_combine      one CTA per token: out[t] = sum_j p[t, j] * (e[t, j] < E ? y[row[t, j]] : x[t]) + g[t] * y_shared[t], summed in the
//                    order written, in fp32; y holds the expert outputs of the assignments sorted by expert, row[t, j] the place of
//                    assignment (t, j) in that order; outputs e >= E are identity experts.  `unit`: every p is 1 (the routing weight
//                    went into the experts' inputs); without g the shared expert's output is added as it is.
//   moe_dispatch     up to 1024 assignments: their places in the order sorted by expert and the experts' row offsets, one CTA.
//   moe_gather       the token rows copied into that order, optionally times the assignment's routing weight (fp32 product).
#include "anytype.cuh"

namespace {

using rb::ld_any;

constexpr int kMaxOutputs = 64, kMaxTop = 8;

__global__ void __launch_bounds__(128) softmax_router_kernel(const void* __restrict__ x, int64_t ldx, int dtx, const void* __restrict__ w, int dtw,
                                                             const void* __restrict__ corr, int dtc, const void* __restrict__ u, int dtu,
                                                             float* __restrict__ probs, int64_t* __restrict__ idx, float* __restrict__ gate,
                                                             int64_t T, int K, int R, int k, int renorm, int sigmoid) {
  __shared__ float s_part[4][kMaxOutputs + 1];
  __shared__ float s_z[kMaxOutputs];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int64_t xb = t * ldx;
  const bool vec = (K & 3) == 0 && (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                   (u == nullptr || (reinterpret_cast<uintptr_t>(u) & 15) == 0);
  const int n_rows = R + (u != nullptr ? 1 : 0);           // row R: the gate vector
  for (int e0 = 0; e0 < n_rows; e0 += 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (vec) {
#pragma unroll 2
      for (int c = threadIdx.x * 4; c < K; c += 512) {
        const float4 xv = rb::ld4_any(x, dtx, xb + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int e = e0 + j;
          if (e < n_rows) {
            const float4 wv = e < R ? rb::ld4_any(w, dtw, (int64_t)e * K + c) : rb::ld4_any(u, dtu, c);
            acc[j] = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc[j]))));
          }
        }
      }
    } else {
      for (int c = threadIdx.x; c < K; c += 128) {
        const float xv = ld_any(x, dtx, xb + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int e = e0 + j;
          if (e < n_rows) acc[j] = fmaf(xv, e < R ? ld_any(w, dtw, (int64_t)e * K + c) : ld_any(u, dtu, c), acc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = rb::warp_sum(acc[j]);
      if (lane == 0 && e0 + j < n_rows) s_part[wid][e0 + j] = v;
    }
  }
  __syncthreads();
  if (wid != 0) return;
  for (int e = lane; e < n_rows; e += 32) {
    const float v = (s_part[0][e] + s_part[1][e]) + (s_part[2][e] + s_part[3][e]);
    if (e < R) s_z[e] = v;
    else gate[t] = 1.f / (1.f + expf(-v));
  }
  __syncwarp();
  // softmax over the R outputs: lane l holds outputs l and l + 32
  const float z0 = lane < R ? s_z[lane] : -INFINITY, z1 = lane + 32 < R ? s_z[lane + 32] : -INFINITY;
  const float mx = rb::warp_max(fmaxf(z0, z1));
  const float e0v = lane < R ? expf(z0 - mx) : 0.f, e1v = lane + 32 < R ? expf(z1 - mx) : 0.f;
  const float den = rb::warp_sum(e0v + e1v);
  const float s0 = sigmoid ? 1.f / (1.f + expf(-z0)) : e0v / den, s1 = sigmoid ? 1.f / (1.f + expf(-z1)) : e1v / den;
  float c0 = lane < R ? s0 + (corr != nullptr ? ld_any(corr, dtc, lane) : 0.f) : -INFINITY;
  float c1 = lane + 32 < R ? s1 + (corr != nullptr ? ld_any(corr, dtc, lane + 32) : 0.f) : -INFINITY;
  float sel_p[kMaxTop];
  int sel_e[kMaxTop];
  float tot = 0.f;
  for (int j = 0; j < k; ++j) {
    // the largest remaining choice score; among equal ones the lowest output
    float best = c0 >= c1 ? c0 : c1;
    int be = c0 >= c1 ? lane : lane + 32;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    const float ps = __shfl_sync(0xffffffffu, be < 32 ? s0 : s1, be & 31);
    sel_p[j] = ps; sel_e[j] = be; tot += ps;
    if (be == lane) c0 = -INFINITY;
    if (be == lane + 32) c1 = -INFINITY;
  }
  if (lane == 0) {
    for (int j = 0; j < k; ++j) {
      probs[t * k + j] = renorm ? sel_p[j] / tot : sel_p[j];
      idx[t * k + j] = sel_e[j];
    }
  }
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const void* __restrict__ y, int dty, const void* __restrict__ x, int64_t ldx, int dtx,
                                                          const int64_t* __restrict__ row, const float* __restrict__ probs,
                                                          const int64_t* __restrict__ idx, const void* __restrict__ ysh, int dts,
                                                          const float* __restrict__ gate, void* __restrict__ out, int dto, int H, int k, int E,
                                                          int unit) {
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  float p[kMaxTop];
  int64_t r[kMaxTop];
  for (int j = 0; j < k; ++j) {
    p[j] = unit ? 1.f : probs[t * k + j];
    r[j] = idx[t * k + j] < E ? row[t * k + j] : -1;
  }
  const float g = gate != nullptr ? gate[t] : 1.f;
  const bool vec = (H & 3) == 0 && (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ysh == nullptr || (reinterpret_cast<uintptr_t>(ysh) & 15) == 0);
  if (vec) {
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < k; ++j) {
        const float4 v = r[j] >= 0 ? rb::ld4_any(y, dty, r[j] * H + c) : rb::ld4_any(x, dtx, t * ldx + c);
        a.x += v.x * p[j]; a.y += v.y * p[j]; a.z += v.z * p[j]; a.w += v.w * p[j];
      }
      if (ysh != nullptr) {
        const float4 v = rb::ld4_any(ysh, dts, t * (int64_t)H + c);
        a.x += v.x * g; a.y += v.y * g; a.z += v.z * g; a.w += v.w * g;
      }
      rb::st4_any(out, dto, t * (int64_t)H + c, a);
    }
    return;
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < k; ++j) a += (r[j] >= 0 ? ld_any(y, dty, r[j] * H + c) : ld_any(x, dtx, t * ldx + c)) * p[j];
    if (ysh != nullptr) a += ld_any(ysh, dts, t * (int64_t)H + c) * g;
    rb::st_any(out, dto, t * (int64_t)H + c, a);
  }
}

// Small batches (N = T k assignments <= 1024): the place of every assignment in the order sorted by expert (stable: equal experts keep
// the order of (token, choice)) and the row offsets of the first E experts, by one CTA, without a sort.
__global__ void __launch_bounds__(1024) moe_dispatch_kernel(const int64_t* __restrict__ idx, int64_t* __restrict__ back, int* __restrict__ offsets,
                                                            int N, int E, int R) {
  __shared__ int s_e[1024];
  __shared__ int s_cnt[kMaxOutputs], s_start[kMaxOutputs + 1];
  const int i = threadIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  if (i < R) s_cnt[i] = 0;
  if (i < N) s_e[i] = (int)idx[i];
  __syncthreads();
  int rank = 0, e = 0;
  if (i < N) {
    e = s_e[i];
    for (int j = 0; j < i; ++j) rank += s_e[j] == e ? 1 : 0;
    atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (i == 0) {
    int acc = 0;
    for (int x = 0; x < R; ++x) { s_start[x] = acc; acc += s_cnt[x]; }
    s_start[R] = acc;
  }
  __syncthreads();
  if (i < N) back[i] = s_start[e] + rank;
  if (i <= E) offsets[i] = s_start[i];
}

// xs[row[i]] = x[i / k] (* scale[i]): the token rows laid out in the sorted order
__global__ void __launch_bounds__(128) moe_gather_kernel(const void* __restrict__ x, int64_t ldx, int dt, const int64_t* __restrict__ row,
                                                         const float* __restrict__ scale, void* __restrict__ xs, int H, int k) {
  const int64_t i = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int64_t src = (i / k) * ldx, dst = row[i] * (int64_t)H;
  const int es = rb::elt_size(dt);
  if (scale != nullptr) {
    const float sc = scale[i];
    if ((H & 3) == 0 && (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(xs) & 15) == 0) {
      for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        const float4 v = rb::ld4_any(x, dt, src + c);
        rb::st4_any(xs, dt, dst + c, make_float4(v.x * sc, v.y * sc, v.z * sc, v.w * sc));
      }
      return;
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) rb::st_any(xs, dt, dst + c, ld_any(x, dt, src + c) * sc);
    return;
  }
  if (((H * es) & 15) == 0 && ((ldx * es) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(xs) & 15) == 0) {
    const uint4* a = reinterpret_cast<const uint4*>(static_cast<const char*>(x) + src * es);
    uint4* b = reinterpret_cast<uint4*>(static_cast<char*>(xs) + dst * es);
    for (int c = threadIdx.x; c < H * es / 16; c += blockDim.x) b[c] = a[c];
    return;
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) rb::st_any(xs, dt, dst + c, ld_any(x, dt, src + c));
}

}  // namespace

extern "C" int rb_softmax_router(const void* x, int64_t ldx, int dtx, const void* w, int dtw, const void* corr, int dtc, const void* u, int dtu,
                                 float* probs, int64_t* idx, float* gate, int64_t T, int K, int R, int k, int renorm, int sigmoid, cudaStream_t s) {
  if (T == 0) return 0;
  if (R < 1 || R > kMaxOutputs || k < 1 || k > kMaxTop || k > R) return -1;
  return rb::launch_pdl(softmax_router_kernel, dim3((unsigned)T), dim3(128), 0, s, x, ldx, dtx, w, dtw, corr, dtc, u, dtu,
                        probs, idx, gate, T, K, R, k, renorm, sigmoid) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_moe_combine(const void* y, int dty, const void* x, int64_t ldx, int dtx, const int64_t* row, const float* probs, const int64_t* idx,
                              const void* ysh, int dts, const float* gate, void* out, int dto, int64_t T, int H, int k, int E, int unit,
                              cudaStream_t s) {
  if (T == 0) return 0;
  if (k < 1 || k > kMaxTop) return -1;
  return rb::launch_pdl(moe_combine_kernel, dim3((unsigned)T), dim3(256), 0, s, y, dty, x, ldx, dtx, row, probs, idx, ysh, dts, gate, out, dto, H, k,
                        E, unit) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_moe_dispatch(const int64_t* idx, int64_t* back, int* offsets, int N, int E, int R, cudaStream_t s) {
  if (N < 1 || N > 1024 || R > kMaxOutputs || E > R) return -1;
  return rb::launch_pdl(moe_dispatch_kernel, dim3(1), dim3(1024), 0, s, idx, back, offsets, N, E, R) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_moe_gather(const void* x, int64_t ldx, int dt, const int64_t* row, const float* scale, void* xs, int64_t N, int H, int k,
                             cudaStream_t s) {
  if (N == 0) return 0;
  return rb::launch_pdl(moe_gather_kernel, dim3((unsigned)N), dim3(128), 0, s, x, ldx, dt, row, scale, xs, H, k) == cudaSuccess ? 0 : 2;
}
