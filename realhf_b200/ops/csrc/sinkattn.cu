// Window attention with a sink (`WindowAttentionConfig`): grouped key / value heads, no rotation.
//
//   score(i, j) = q_i . k_j * scale * temp_h - slope_h * (i - j),   slope_h = 2^(-slope_base (h + 1) / H)
//   visible:      j <= i and (i - j < window or j < keep_first)                (window < 0: every j <= i)
//   weights:      exp(score - m) / (sum_visible exp(score - m) + exp(sink_h - m))   (the sink is a bare logit: key-less, value-less)
//   output:       sum_j w_ij vhat_j * sigmoid(gate_h),   vhat = v / sqrt(mean(v^2) + eps) per head (cached so)
//
// Everything is fp32 arithmetic whatever the storage type (a type code per launch: 0 fp32, 1 bf16, 2 fp16); exact expf (compiled
// without fast-math).  The projection output `qkvg` [T, ld] holds [q (H x d) | k (G x d) | v (G x dv) | gate logits] per row.
// Caches: kc [n_slots, G, rows, d], vc [n_slots, G / vshare, rows, dv]; position p lives in row p when p < keep_first, else in row
// keep_first + (p - keep_first) % (rows - keep_first).  `vshare` consecutive key heads read the same value head (1: a value head
// per key head; 2: the two score maps of differential attention over one set of values), and the projection row then holds
// G / vshare value heads.
//
//   value_norm_store       packed prefill: vhat -> [T, G * dv], and the rows a later decode step can still see -> caches
//   sink_window_prefill    packed prefill over the batch's own keys: CTA = 32 queries x 1 head of one sequence, 32-key tiles in
//                          shared memory, online softmax whose running maximum starts at the sink (denominator 1)
//   qk_head_norm           in place: every query / key head of a row divided by its root mean square, times a weight per section
//   diff_combine           differential attention: o = a1 - lambda a2 per head, o / sqrt(mean(o^2) + eps) * (1 - diff)
//   sink_window_decode     one token per row: CTA = (row, kv head) serving the group's query heads; appends k / vhat, then walks the
//                          visible cache rows in 128-key tiles (one key per thread for the scores, one column per thread for P.V)
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

RB_DEVICE int cache_row(int p, int keep, int rows) {
  const int ring = max(rows - keep, 1);
  return p < keep ? p : keep + (p - keep) % ring;
}

// ------------------------------------------------------------------------------------------------ value norm + cache fill
// one CTA per token; a warp per kv head (looping)
__global__ void __launch_bounds__(128) value_norm_store_kernel(const void* __restrict__ qkvg, int64_t ld, int dt, void* __restrict__ vout,
                                                                void* __restrict__ kc, void* __restrict__ vc, const int* __restrict__ tok_slot,
                                                                const int* __restrict__ pos, const int* __restrict__ remain, int H, int G, int d,
                                                                int dv, int keep, int rows, int do_norm, float eps, int vshare) {
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int64_t base = t * ld;
  const int ok = H * d, ov = ok + G * d;
  int slot = -1, row = 0;
  if (kc != nullptr) {
    slot = tok_slot[t];
    const int p = pos[t];
    if (slot >= 0 && !(p < keep || remain[t] < rows - keep)) slot = -1;   // a row that a later position of this prompt overwrites
    row = cache_row(p, keep, rows);
  }
  const int Gv = G / vshare;
  for (int g = warp; g < Gv; g += nwarp) {
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = ld_any(qkvg, dt, base + ov + g * dv + c); ss += v * v; }
    ss = rb::warp_sum(ss);
    const float r = do_norm ? 1.f / sqrtf(ss / (float)dv + eps) : 1.f;
    const int64_t crow = slot >= 0 ? ((int64_t)slot * Gv + g) * rows + row : 0;
    for (int c = lane; c < dv; c += 32) {
      const float v = ld_any(qkvg, dt, base + ov + g * dv + c) * r;
      if (vout != nullptr) st_any(vout, dt, t * (int64_t)(Gv * dv) + g * dv + c, v);
      if (slot >= 0) st_any(vc, dt, crow * dv + c, v);
    }
  }
  if (slot >= 0)
    for (int g = warp; g < G; g += nwarp) {
      const int64_t crow = ((int64_t)slot * G + g) * rows + row;
      for (int c = lane; c < d; c += 32) st_any(kc, dt, crow * d + c, ld_any(qkvg, dt, base + ok + g * d + c));
    }
}

// ------------------------------------------------------------------------------------------------ packed prefill
constexpr int BQ = 32, BK = 32, kPfThreads = 128;

struct PrefillParams {
  const void* qkvg; int64_t ld;
  const void* vn;            // [T, vld] rows of G / vshare value heads
  void* out;                 // [T, H * dv] in type dto
  const void* temp; const void* sink;   // [H] in the model type, or null
  const int* cu;             // [n_seqs + 1]
  int H, G, d, dv, window, keep, gate, dt;
  float scale, slope_base;
  int vshare, dto; int64_t vld;
};

// NJ = ceil(dv / 32): a thread owns 2 query rows x NJ float4 column groups of the output tile
template <int NJ>
__global__ void __launch_bounds__(kPfThreads) sink_window_prefill_kernel(PrefillParams p) {
  extern __shared__ __align__(16) float smem[];
  const int seq = blockIdx.y, h = blockIdx.z, g = h / (p.H / p.G);
  const int s0 = p.cu[seq], L = p.cu[seq + 1] - s0;
  const int q0 = blockIdx.x * BQ;
  if (q0 >= L) return;
  const int d = p.d, dv = p.dv, dp = (d + 3) & ~3, dvp = NJ * 32;
  const int qs = dp + 4, vs = dvp + 4;                // padded row strides (floats): conflict-free float4 reads
  float* Qs = smem;                                   // [BQ][qs]
  float* Ks = Qs + BQ * qs;                           // [BK][qs]
  float* Vs = Ks + BK * qs;                           // [BK][vs]
  float* Ps = Vs + BK * vs;                           // [BQ][BK + 1]
  const int tid = threadIdx.x, tx = tid & 7, ty = tid >> 3;   // tx: keys tx + 8c of a tile / float4 output groups; ty: 2 query rows
  const int nq = min(BQ, L - q0);
  const int dt = p.dt;
  const int ok = p.H * d;

  for (int idx = tid; idx < BQ * dp; idx += kPfThreads) {
    const int r = idx / dp, e = idx % dp;
    Qs[r * qs + e] = (r < nq && e < d) ? ld_any(p.qkvg, dt, (int64_t)(s0 + q0 + r) * p.ld + h * d + e) : 0.f;
  }
  const float qmul = p.scale * (p.temp ? ld_any(p.temp, dt, h) : 1.f);
  const float slope = p.slope_base >= 0.f ? exp2f(-p.slope_base * (float)(h + 1) / (float)p.H) : 0.f;
  float m[2], l[2], o[2][NJ][4];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (p.sink) { m[r] = ld_any(p.sink, dt, h); l[r] = 1.f; } else { m[r] = -INFINITY; l[r] = 0.f; }
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[r][j][c] = 0.f;
  }
  // key ranges of this query tile: the kept first tokens [0, ka) and the window part [lo, q_last]
  const int q_last = q0 + nq - 1;
  const int lo = p.window < 0 ? 0 : max(0, q0 - p.window + 1);
  const int ka = p.window < 0 ? 0 : min(p.keep, lo);
  const int lo_al = lo / BK * BK;                       // window tiles start on a tile border
  const int n_keep_tiles = RB_CEIL_DIV(min(ka, lo_al), BK);   // keys of [0, ka) below lo_al (the rest falls into window tiles)
  const int n_win_tiles = RB_CEIL_DIV(q_last + 1 - lo_al, BK);

  for (int tile = 0; tile < n_keep_tiles + n_win_tiles; ++tile) {
    const int k0 = tile < n_keep_tiles ? tile * BK : lo_al + (tile - n_keep_tiles) * BK;
    const int kend = tile < n_keep_tiles ? min(ka, lo_al) : q_last + 1;   // keys at or beyond kend are not loaded
    __syncthreads();
    for (int idx = tid; idx < BK * dp; idx += kPfThreads) {
      const int r = idx / dp, e = idx % dp;
      Ks[r * qs + e] = (k0 + r < kend && e < d) ? ld_any(p.qkvg, dt, (int64_t)(s0 + k0 + r) * p.ld + ok + g * d + e) : 0.f;
    }
    for (int idx = tid; idx < BK * dvp; idx += kPfThreads) {
      const int r = idx / dvp, e = idx % dvp;
      Vs[r * vs + e] = (k0 + r < kend && e < dv) ? ld_any(p.vn, dt, (int64_t)(s0 + k0 + r) * p.vld + (g / p.vshare) * dv + e) : 0.f;
    }
    __syncthreads();
    // scores of 2 rows x 4 keys
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int e = 0; e < dp; e += 4) {
      const float4 qa = *reinterpret_cast<const float4*>(Qs + (ty * 2) * qs + e);
      const float4 qb = *reinterpret_cast<const float4*>(Qs + (ty * 2 + 1) * qs + e);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 kk = *reinterpret_cast<const float4*>(Ks + (tx + 8 * c) * qs + e);
        s[0][c] = fmaf(qa.x, kk.x, fmaf(qa.y, kk.y, fmaf(qa.z, kk.z, fmaf(qa.w, kk.w, s[0][c]))));
        s[1][c] = fmaf(qb.x, kk.x, fmaf(qb.y, kk.y, fmaf(qb.z, kk.z, fmaf(qb.w, kk.w, s[1][c]))));
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = q0 + ty * 2 + r;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = k0 + tx + 8 * c;
        const bool vis = j < kend && j <= i && i <= q_last && (p.window < 0 || i - j < p.window || j < p.keep);
        s[r][c] = vis ? s[r][c] * qmul - slope * (float)(i - j) : -INFINITY;
        mx = fmaxf(mx, s[r][c]);
      }
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float mn = fmaxf(m[r], mx);
      const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - mn);
      float ps = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float pr = (s[r][c] == -INFINITY) ? 0.f : expf(s[r][c] - mn);
        Ps[(ty * 2 + r) * (BK + 1) + tx + 8 * c] = pr;
        ps += pr;
      }
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
      l[r] = l[r] * corr + ps;
      m[r] = mn;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[r][j][c] *= corr;
    }
    __syncwarp();   // a row's 8 score lanes and its 8 output lanes are the same lanes of one warp
    const int nk = min(BK, kend - k0);
    for (int kk = 0; kk < nk; ++kk) {
      const float pa = Ps[(ty * 2) * (BK + 1) + kk], pb = Ps[(ty * 2 + 1) * (BK + 1) + kk];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(Vs + kk * vs + j * 32 + tx * 4);
        o[0][j][0] = fmaf(pa, v.x, o[0][j][0]); o[0][j][1] = fmaf(pa, v.y, o[0][j][1]);
        o[0][j][2] = fmaf(pa, v.z, o[0][j][2]); o[0][j][3] = fmaf(pa, v.w, o[0][j][3]);
        o[1][j][0] = fmaf(pb, v.x, o[1][j][0]); o[1][j][1] = fmaf(pb, v.y, o[1][j][1]);
        o[1][j][2] = fmaf(pb, v.z, o[1][j][2]); o[1][j][3] = fmaf(pb, v.w, o[1][j][3]);
      }
    }
  }
  const int og = p.H * d + p.G * d + p.G / p.vshare * dv;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = q0 + ty * 2 + r;
    if (i > q_last) continue;
    const int64_t t = s0 + i;
    float f = l[r] > 0.f ? 1.f / l[r] : 0.f;
    if (p.gate) f *= 1.f / (1.f + expf(-ld_any(p.qkvg, dt, t * p.ld + og + h)));
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col = j * 32 + tx * 4 + c;
        if (col < dv) st_any(p.out, p.dto, t * (int64_t)(p.H * dv) + h * dv + col, o[r][j][c] * f);
      }
  }
}

// ------------------------------------------------------------------------------------------------ query / key head norm, differential combine
// a warp per (row, head); heads [0, nq) take weight wq, heads [nq, nq + nk) weight wk; the heads are consecutive in the row
__global__ void __launch_bounds__(128) qk_head_norm_kernel(void* __restrict__ x, int64_t ld, int dt, const void* __restrict__ wq,
                                                           const void* __restrict__ wk, int64_t n_rows, int nq, int nk, int d, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  rb::pdl_trigger();
  rb::pdl_wait();
  if (id >= n_rows * (nq + nk)) return;
  const int64_t t = id / (nq + nk);
  const int h = (int)(id % (nq + nk));
  const void* w = h < nq ? wq : wk;
  const int64_t base = t * ld + (int64_t)h * d;
  float ss = 0.f;
  if ((d & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {      // 4 elements per access
    for (int c = lane * 4; c < d; c += 128) { const float4 v = rb::ld4_any(x, dt, base + c); ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    ss = rb::warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)d + eps);
    for (int c = lane * 4; c < d; c += 128) {
      const float4 v = rb::ld4_any(x, dt, base + c);
      rb::st4_any(x, dt, base + c, make_float4(v.x * r * ld_any(w, dt, c), v.y * r * ld_any(w, dt, c + 1), v.z * r * ld_any(w, dt, c + 2), v.w * r * ld_any(w, dt, c + 3)));
    }
    return;
  }
  for (int c = lane; c < d; c += 32) { const float v = ld_any(x, dt, base + c); ss += v * v; }
  ss = rb::warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)d + eps);
  for (int c = lane; c < d; c += 32) st_any(x, dt, base + c, ld_any(x, dt, base + c) * r * ld_any(w, dt, c));
}

// a [T, G, 2, per, dv] (the attention outputs of both maps, query heads grouped by key head), out [T, H * dv], H = G * per
__global__ void __launch_bounds__(128) diff_combine_kernel(const void* __restrict__ a, int dta, const float* __restrict__ lam, void* __restrict__ out,
                                                           int dto, int64_t n_rows, int H, int G, int dv, float diff, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  rb::pdl_trigger();
  rb::pdl_wait();
  if (id >= n_rows * H) return;
  const int64_t t = id / H;
  const int h = (int)(id % H), per = H / G, g = h / per, hh = h % per;
  const int64_t b1 = (t * 2 * H + (int64_t)(g * 2) * per + hh) * dv, b2 = b1 + (int64_t)per * dv;
  const float l = lam[0];
  float ss = 0.f;
  if ((dv & 3) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {   // 4 elements per access
    for (int c = lane * 4; c < dv; c += 128) {
      const float4 x = rb::ld4_any(a, dta, b1 + c), y = rb::ld4_any(a, dta, b2 + c);
      const float o0 = x.x - l * y.x, o1 = x.y - l * y.y, o2 = x.z - l * y.z, o3 = x.w - l * y.w;
      ss += o0 * o0 + o1 * o1 + o2 * o2 + o3 * o3;
    }
    ss = rb::warp_sum(ss);
    const float r = (1.f - diff) / sqrtf(ss / (float)dv + eps);
    for (int c = lane * 4; c < dv; c += 128) {
      const float4 x = rb::ld4_any(a, dta, b1 + c), y = rb::ld4_any(a, dta, b2 + c);
      rb::st4_any(out, dto, id * dv + c, make_float4((x.x - l * y.x) * r, (x.y - l * y.y) * r, (x.z - l * y.z) * r, (x.w - l * y.w) * r));
    }
    return;
  }
  for (int c = lane; c < dv; c += 32) { const float o = ld_any(a, dta, b1 + c) - l * ld_any(a, dta, b2 + c); ss += o * o; }
  ss = rb::warp_sum(ss);
  const float r = (1.f - diff) / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) st_any(out, dto, id * dv + c, (ld_any(a, dta, b1 + c) - l * ld_any(a, dta, b2 + c)) * r);
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int kDecThreads = 128, kMaxRep = 8, kMaxColsPerThread = 2;   // dv <= 256

struct DecodeParams {
  const void* qkvg; int64_t ld;
  void* out; const void* temp; const void* sink;
  void* kc; void* vc;
  const int* lens; const int* slots;
  int H, G, d, dv, rows, window, keep, gate, do_norm, dt;
  float scale, slope_base, eps;
  int vshare, dto;
};

__global__ void __launch_bounds__(kDecThreads) sink_window_decode_kernel(DecodeParams p) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // blockIdx.z: a chunk of up to kMaxRep query heads of the group (every chunk's CTA appends the same new row)
  const int group = p.H / p.G, h0 = g * group + blockIdx.z * kMaxRep, rep = min(kMaxRep, group - blockIdx.z * kMaxRep);
  const int d = p.d, dv = p.dv, dt = p.dt;
  float* qs = smem;                         // [rep][d], scaled by scale * temp
  float* ps = qs + rep * d;                 // [rep][kDecThreads]
  float* red = ps + rep * kDecThreads;      // [rep][4] warp partials, then [rep] results at red + rep * 4
  float* vnew = red + rep * 5;              // [dv]
  int* rws = reinterpret_cast<int*>(vnew + dv);   // [kDecThreads] cache rows of the tile's keys
  const int slot = p.slots ? p.slots[b] : b;
  const int n = p.lens[slot];               // the new token's position
  const int64_t base = (int64_t)b * p.ld;
  const int gv = g / p.vshare, Gv = p.G / p.vshare;
  const int ok = p.H * d, ov = ok + p.G * d, og = ov + Gv * dv;
  const int64_t cbase = ((int64_t)slot * p.G + g) * p.rows, vbase = ((int64_t)slot * Gv + gv) * p.rows;

  for (int idx = tid; idx < rep * d; idx += kDecThreads) {
    const int h = h0 + idx / d;
    qs[idx] = ld_any(p.qkvg, dt, base + h * d + idx % d) * (p.scale * (p.temp ? ld_any(p.temp, dt, h) : 1.f));
  }
  // append the new key and normalised value (fp32 statistics; the stored value is what later steps read)
  {
    float ss = 0.f;
    for (int c = tid; c < dv; c += kDecThreads) { const float v = ld_any(p.qkvg, dt, base + ov + gv * dv + c); vnew[c] = v; ss += v * v; }
    ss = rb::block_reduce<false>(ss, red);
    const float r = p.do_norm ? 1.f / sqrtf(ss / (float)dv + p.eps) : 1.f;
    const int nr = cache_row(n, p.keep, p.rows);
    const int64_t row = cbase + nr, vrow_new = vbase + nr;   // (CTAs that share a value head write the same values)
    for (int c = tid; c < dv; c += kDecThreads) st_any(p.vc, dt, vrow_new * dv + c, vnew[c] * r);
    for (int c = tid; c < d; c += kDecThreads) st_any(p.kc, dt, row * d + c, ld_any(p.qkvg, dt, base + ok + g * d + c));
  }
  __syncthreads();   // the CTA's own global writes are visible to its threads from here on

  const int lo = p.window < 0 ? 0 : max(0, n - p.window + 1);
  const int ka = p.window < 0 ? 0 : min(p.keep, lo);
  const int nk = ka + (n - lo + 1);         // visible keys: positions [0, ka) and [lo, n]
  float m[kMaxRep], l[kMaxRep], acc[kMaxRep][kMaxColsPerThread];
#pragma unroll
  for (int r = 0; r < kMaxRep; ++r) {
    if (r < rep && p.sink) { m[r] = ld_any(p.sink, dt, h0 + r); l[r] = 1.f; } else { m[r] = -INFINITY; l[r] = 0.f; }
#pragma unroll
    for (int c = 0; c < kMaxColsPerThread; ++c) acc[r][c] = 0.f;
  }
  const bool vec_k = (d % 4 == 0);
  for (int t0 = 0; t0 < nk; t0 += kDecThreads) {
    const int idx = t0 + tid;
    const bool have = idx < nk;
    const int j = have ? (idx < ka ? idx : lo + idx - ka) : 0;
    float s[kMaxRep];
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r) s[r] = 0.f;
    if (have) {
      const int jr = cache_row(j, p.keep, p.rows);
      rws[tid] = jr;
      const int64_t krow = (cbase + jr) * d;
      if (vec_k) {
        for (int e = 0; e < d; e += 4) {
          const float4 kk = rb::ld4_any(p.kc, dt, krow + e);
#pragma unroll
          for (int r = 0; r < kMaxRep; ++r)
            if (r < rep) {
              const float4 qq = *reinterpret_cast<const float4*>(qs + r * d + e);
              s[r] = fmaf(qq.x, kk.x, fmaf(qq.y, kk.y, fmaf(qq.z, kk.z, fmaf(qq.w, kk.w, s[r]))));
            }
        }
      } else {
        for (int e = 0; e < d; ++e) {
          const float kk = ld_any(p.kc, dt, krow + e);
#pragma unroll
          for (int r = 0; r < kMaxRep; ++r)
            if (r < rep) s[r] = fmaf(qs[r * d + e], kk, s[r]);
        }
      }
    }
    // tile maximum per head -> running maximum, weights into shared memory
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r)
      if (r < rep) {
        const float slope = p.slope_base >= 0.f ? exp2f(-p.slope_base * (float)(h0 + r + 1) / (float)p.H) : 0.f;
        s[r] = have ? s[r] - slope * (float)(n - j) : -INFINITY;
        const float wm = rb::warp_max(s[r]);
        if (lane == 0) red[r * 4 + warp] = wm;
      }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r)
      if (r < rep) {
        const float tm = fmaxf(fmaxf(red[r * 4], red[r * 4 + 1]), fmaxf(red[r * 4 + 2], red[r * 4 + 3]));
        const float mn = fmaxf(m[r], tm);
        const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - mn);
        const float pr = have ? expf(s[r] - mn) : 0.f;
        ps[r * kDecThreads + tid] = pr;
        l[r] *= corr;
#pragma unroll
        for (int c = 0; c < kMaxColsPerThread; ++c) acc[r][c] *= corr;
        m[r] = mn;
      }
    __syncthreads();
    const int cnt = min(kDecThreads, nk - t0);
    // denominators: every thread adds the tile's weights in the same order (no second reduction needed)
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r)
      if (r < rep) {
        float sum = 0.f;
        for (int k = 0; k < cnt; ++k) sum += ps[r * kDecThreads + k];
        l[r] += sum;
      }
    for (int k = 0; k < cnt; ++k) {
      const int64_t vrow = (vbase + rws[k]) * dv;
#pragma unroll
      for (int c = 0; c < kMaxColsPerThread; ++c) {
        const int col = tid + c * kDecThreads;
        if (col < dv) {
          const float v = ld_any(p.vc, dt, vrow + col);
#pragma unroll
          for (int r = 0; r < kMaxRep; ++r)
            if (r < rep) acc[r][c] = fmaf(ps[r * kDecThreads + k], v, acc[r][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < kMaxRep; ++r)
    if (r < rep) {
      const int h = h0 + r;
      float f = l[r] > 0.f ? 1.f / l[r] : 0.f;
      if (p.gate) f *= 1.f / (1.f + expf(-ld_any(p.qkvg, dt, base + og + h)));
#pragma unroll
      for (int c = 0; c < kMaxColsPerThread; ++c) {
        const int col = tid + c * kDecThreads;
        if (col < dv) st_any(p.out, p.dto, (int64_t)b * (p.H * dv) + h * dv + col, acc[r][c] * f);
      }
    }
}

// ------------------------------------------------------------------------------------------------ decode, 16-bit fast path
// Equal query / value head size HD of 64 or 128, 16-bit storage: the streaming design of the dense-cache decode kernel
// (attn_decode.cu).  A group of HD / 8 lanes owns one cache row at a time with 16-byte loads, REP query heads share every load,
// the loop is unrolled x4, the softmax exponentials use the fast intrinsic (fp32 arithmetic; the all-fp32 kernel above keeps expf),
// launches are programmatic dependent launches like the dense kernel's, and the visible keys are cut into `splits` ranges (grid.z)
// whose partial (max, sum, acc) are merged
// by a second kernel, so that a batch of few rows still fills the GPU.  The visible keys are indexed 0 .. nk - 1 (kept first
// tokens, then the window); index -> cache row needs no division (the ring wraps at most once inside a window).
constexpr int kFastWarps = 4, kFastThreads = kFastWarps * 32;

template <typename T> RB_DEVICE void f_load8(const T* p, float* f) {
  rb::Pack<T, 8> v = *reinterpret_cast<const rb::Pack<T, 8>*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = rb::to_f(v.v[i]);
}
template <typename T> RB_DEVICE void f_store8(T* p, const float* f) {
  rb::Pack<T, 8> v;
#pragma unroll
  for (int i = 0; i < 8; ++i) v.v[i] = rb::from_f<T>(f[i]);
  *reinterpret_cast<rb::Pack<T, 8>*>(p) = v;
}

struct FastParams {
  DecodeParams d;
  float* part_acc;   // [B, H, splits, HD]
  float* part_ml;    // [B, H, splits, 2]
  int splits;
};

template <typename T, int HD, int REP>
__global__ void __launch_bounds__(kFastThreads) sink_window_decode_fast_kernel(FastParams fp) {
  const DecodeParams& p = fp.d;
  constexpr int LPR = HD / 8, RPW = 32 / LPR;
  const int b = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane % LPR, rsel = lane / LPR;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int slot = p.slots ? p.slots[b] : b;
  const int n = p.lens[slot];
  const T* row_in = reinterpret_cast<const T*>(p.qkvg) + (int64_t)b * p.ld;
  const int Gv = p.G / p.vshare, gv = g / p.vshare;
  const int ok = p.H * HD, ov = ok + p.G * HD, og = ov + Gv * HD;
  T* kc = reinterpret_cast<T*>(p.kc) + ((int64_t)slot * p.G + g) * p.rows * HD;
  T* vc = reinterpret_cast<T*>(p.vc) + ((int64_t)slot * Gv + gv) * p.rows * HD;   // (CTAs that share a value head append the same values)

  float q[REP][8], slope[REP], kn[8], vn[8];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const int h = g * REP + r;
    f_load8(row_in + h * HD + sub * 8, q[r]);
    const float mul = p.scale * (p.temp ? rb::to_f(reinterpret_cast<const T*>(p.temp)[h]) : 1.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[r][i] *= mul;
    slope[r] = p.slope_base >= 0.f ? exp2f(-p.slope_base * (float)(h + 1) / (float)p.H) : 0.f;
  }
  f_load8(row_in + ok + g * HD + sub * 8, kn);
  f_load8(row_in + ov + gv * HD + sub * 8, vn);
  if (p.do_norm) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(vn[i], vn[i], ss);
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, LPR);
    const float rs = 1.f / sqrtf(ss / (float)HD + p.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) vn[i] = rb::to_f(rb::from_f<T>(vn[i] * rs));     // as later steps will read it from the cache
  }
  const int ring = max(p.rows - p.keep, 1);
  const int lo = p.window < 0 ? 0 : max(0, n - p.window + 1);
  const int ka = p.window < 0 ? 0 : min(p.keep, lo);
  const bool flat = lo < p.keep;                       // every visible position still lives in row = position
  const int r_lo = flat ? 0 : (lo - p.keep) % ring;
  auto pos_of = [&](int idx) { return idx < ka ? idx : lo + idx - ka; };
  auto row_of = [&](int idx) {
    if (idx < ka) return idx;
    const int w = idx - ka;
    if (flat) return lo + w;
    const int rr = r_lo + w;
    return p.keep + (rr >= ring ? rr - ring : rr);
  };
  const int nk = ka + (n - lo + 1);                    // the last index is the new token itself
  if (split == 0 && warp == 0 && rsel == 0) {
    const int64_t rn = row_of(nk - 1);
    f_store8(kc + rn * HD + sub * 8, kn);
    f_store8(vc + rn * HD + sub * 8, vn);
  }
  const int cached = nk - 1;
  const int per = RB_CEIL_DIV(cached, fp.splits);
  const int i0 = min(cached, split * per), i1 = min(cached, i0 + per);

  float m[REP], l[REP], acc[REP][8];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
    if (p.sink && split == 0 && warp == 0 && rsel == 0) { m[r] = rb::to_f(reinterpret_cast<const T*>(p.sink)[g * REP + r]); l[r] = 1.f; }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
  }
  const unsigned gmask = (LPR == 32) ? 0xffffffffu : (((1u << LPR) - 1u) << (rsel * LPR));
  auto consume = [&](const float* kf, const float* vf, int idx) {
    const float dist = (float)(n - pos_of(idx));
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(q[r][i], kf[i], s);
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(gmask, s, o, LPR);
      s -= slope[r] * dist;
      const float mn = fmaxf(m[r], s);
      const float corr = (m[r] == -INFINITY) ? 0.f : __expf(m[r] - mn), pr = __expf(s - mn);
      l[r] = l[r] * corr + pr;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(acc[r][i], corr, pr * vf[i]);
      m[r] = mn;
    }
  };
  constexpr int UNROLL = 4;
  const int step = kFastWarps * RPW;
  int s0 = i0 + warp * RPW + rsel;
  for (; s0 + (UNROLL - 1) * step < i1; s0 += UNROLL * step) {
    float kf[UNROLL][8], vf[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t rr = row_of(s0 + u * step);
      f_load8(kc + rr * HD + sub * 8, kf[u]);
      f_load8(vc + rr * HD + sub * 8, vf[u]);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) consume(kf[u], vf[u], s0 + u * step);
  }
  for (; s0 < i1; s0 += step) {
    float kf[8], vf[8];
    const int64_t rr = row_of(s0);
    f_load8(kc + rr * HD + sub * 8, kf);
    f_load8(vc + rr * HD + sub * 8, vf);
    consume(kf, vf, s0);
  }
  if (split == fp.splits - 1 && warp == 0 && rsel == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) kn[i] = rb::to_f(rb::from_f<T>(kn[i]));
    consume(kn, vn, nk - 1);
  }
  __syncwarp();
  __shared__ float sm_acc[kFastWarps][REP][HD];
  __shared__ float sm_m[kFastWarps][REP], sm_l[kFastWarps][REP];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[r], o), l2 = __shfl_xor_sync(0xffffffffu, l[r], o);
      const float mn = fmaxf(m[r], m2);
      const float c1 = (m[r] == -INFINITY) ? 0.f : __expf(m[r] - mn), c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
      l[r] = l[r] * c1 + l2 * c2;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a2 = __shfl_xor_sync(0xffffffffu, acc[r][i], o);
        acc[r][i] = acc[r][i] * c1 + a2 * c2;
      }
      m[r] = mn;
    }
    if (rsel == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_acc[warp][r][sub * 8 + i] = acc[r][i];
      if (sub == 0) { sm_m[warp][r] = m[r]; sm_l[warp][r] = l[r]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < REP * HD; idx += kFastThreads) {
    const int r = idx / HD, c = idx % HD;
    float mg = -INFINITY;
#pragma unroll
    for (int w = 0; w < kFastWarps; ++w) mg = fmaxf(mg, sm_m[w][r]);
    float lg = 0.f, ag = 0.f;
#pragma unroll
    for (int w = 0; w < kFastWarps; ++w) {
      const float cf = (sm_m[w][r] == -INFINITY) ? 0.f : __expf(sm_m[w][r] - mg);
      lg += sm_l[w][r] * cf;
      ag += sm_acc[w][r][c] * cf;
    }
    const int h = g * REP + r;
    if (fp.splits == 1) {
      float f = lg > 0.f ? 1.f / lg : 0.f;
      if (p.gate) f *= 1.f / (1.f + expf(-rb::to_f(row_in[og + h])));
      reinterpret_cast<T*>(p.out)[(int64_t)b * p.H * HD + (int64_t)h * HD + c] = rb::from_f<T>(ag * f);
    } else {
      const int64_t o = ((int64_t)b * p.H + h) * fp.splits + split;
      fp.part_acc[o * HD + c] = ag;
      if (c == 0) { fp.part_ml[o * 2] = mg; fp.part_ml[o * 2 + 1] = lg; }
    }
  }
}

template <typename T, int HD>
__global__ void sink_window_decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, const T* __restrict__ qkvg,
                                                int64_t ld, int og, int H, int gate, T* __restrict__ out, int splits) {
  const int64_t bh = blockIdx.x;
  const int c = threadIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  float mg = -INFINITY;
  for (int s = 0; s < splits; ++s) mg = fmaxf(mg, part_ml[(bh * splits + s) * 2]);
  float lg = 0.f, ag = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(bh * splits + s) * 2];
    const float cf = (ms == -INFINITY) ? 0.f : expf(ms - mg);
    lg += part_ml[(bh * splits + s) * 2 + 1] * cf;
    ag += part_acc[(bh * splits + s) * HD + c] * cf;
  }
  float f = lg > 0.f ? 1.f / lg : 0.f;
  if (gate) f *= 1.f / (1.f + expf(-rb::to_f(qkvg[(bh / H) * ld + og + (bh % H)])));
  out[bh * HD + c] = rb::from_f<T>(ag * f);
}

template <typename T, int HD>
int launch_fast(const FastParams& fp, int B, cudaStream_t s) {
  const DecodeParams& p = fp.d;
  dim3 grid(B, p.G, fp.splits);
#define RB_L(REP) rb::launch_pdl(sink_window_decode_fast_kernel<T, HD, REP>, grid, dim3(kFastThreads), 0, s, fp)
  switch (p.H / p.G) {
    case 1: RB_L(1); break;
    case 2: RB_L(2); break;
    case 4: RB_L(4); break;
    case 8: RB_L(8); break;
    default: return -1;
  }
#undef RB_L
  if (fp.splits > 1)
    rb::launch_pdl(sink_window_decode_merge_kernel<T, HD>, dim3(B * p.H), dim3(HD), 0, s, (const float*)fp.part_acc, (const float*)fp.part_ml,
                   reinterpret_cast<const T*>(p.qkvg), p.ld, p.H * HD + p.G * HD + p.G / p.vshare * HD, p.H, p.gate, reinterpret_cast<T*>(p.out), fp.splits);
  return 0;
}

}  // namespace

extern "C" int rb_value_norm_store(const void* qkvg, int64_t ld, int dt, void* vout, void* kc, void* vc, const int* tok_slot, const int* pos,
                                   const int* remain, int64_t T, int H, int G, int d, int dv, int keep, int rows, int do_norm, float eps,
                                   int vshare, cudaStream_t s) {
  if (T == 0) return 0;
  if (vshare < 1 || G % vshare) return -1;
  value_norm_store_kernel<<<(unsigned)T, 128, 0, s>>>(qkvg, ld, dt, vout, kc, vc, tok_slot, pos, remain, H, G, d, dv, keep, rows, do_norm, eps, vshare);
  return 0;
}

extern "C" int rb_sink_window_prefill(const void* qkvg, int64_t ld, const void* vn, void* out, const void* temp, const void* sink, const int* cu,
                                      int n_seqs, int max_seqlen, int H, int G, int d, int dv, float scale, int window, int keep, float slope_base,
                                      int gate, int dt, int vshare, int64_t vld, int dto, cudaStream_t s) {
  if (n_seqs == 0 || max_seqlen == 0) return 0;
  if (dv > 256 || d > 512 || H % G || vshare < 1 || G % vshare) return -1;
  PrefillParams p{qkvg, ld, vn, out, temp, sink, cu, H, G, d, dv, window, keep, gate, dt, scale, slope_base, vshare, dto, vld};
  const int nj = dv <= 32 ? 1 : dv <= 64 ? 2 : dv <= 128 ? 4 : 8;
  const int dp = (d + 3) & ~3;
  const size_t smem = sizeof(float) * ((size_t)(BQ + BK) * (dp + 4) + (size_t)BK * (nj * 32 + 4) + (size_t)BQ * (BK + 1));
  dim3 grid(RB_CEIL_DIV(max_seqlen, BQ), n_seqs, H);
#define RB_L(NJ)                                                                                                          \
  {                                                                                                                       \
    if (smem > 48 * 1024) cudaFuncSetAttribute(sink_window_prefill_kernel<NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    sink_window_prefill_kernel<NJ><<<grid, kPfThreads, smem, s>>>(p);                                                     \
  }
  switch (nj) {
    case 1: RB_L(1); break;
    case 2: RB_L(2); break;
    case 4: RB_L(4); break;
    default: RB_L(8); break;
  }
#undef RB_L
  return 0;
}

extern "C" int rb_sink_window_decode(const void* qkvg, int64_t ld, void* out, const void* temp, const void* sink, void* kc, void* vc,
                                     const int* lens, const int* slots, int B, int H, int G, int d, int dv, int rows, float scale, int window,
                                     int keep, float slope_base, int gate, int do_norm, float eps, int dt, int vshare, int dto, cudaStream_t s) {
  if (B == 0) return 0;
  const int rep = min(H / G, kMaxRep);
  if (H % G || dv > kDecThreads * kMaxColsPerThread || vshare < 1 || G % vshare) return -1;
  DecodeParams p{qkvg, ld, out, temp, sink, kc, vc, lens, slots, H, G, d, dv, rows, window, keep, gate, do_norm, dt, scale, slope_base, eps, vshare, dto};
  const size_t smem = sizeof(float) * ((size_t)rep * d + (size_t)rep * kDecThreads + rep * 5 + 32 + dv + kDecThreads);
  if (smem > 48 * 1024) cudaFuncSetAttribute(sink_window_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  sink_window_decode_kernel<<<dim3(B, G, RB_CEIL_DIV(H / G, kMaxRep)), kDecThreads, smem, s>>>(p);
  return 0;
}

// 16-bit fast path of the decode form (dt 1 / 2, d == dv in {64, 128}, H / G in {1, 2, 4, 8}, 16-byte aligned rows); part_acc
// [B, H, splits, d] and part_ml [B, H, splits, 2] fp32 are scratch for splits > 1.  Returns -1 for shapes it does not take.
extern "C" int rb_sink_window_decode_fast(const void* qkvg, int64_t ld, void* out, const void* temp, const void* sink, void* kc, void* vc,
                                          const int* lens, const int* slots, float* part_acc, float* part_ml, int splits, int B, int H, int G, int d,
                                          int rows, float scale, int window, int keep, float slope_base, int gate, int do_norm, float eps, int dt,
                                          int vshare, cudaStream_t s) {
  if (B == 0) return 0;
  if ((dt != 1 && dt != 2) || (d != 64 && d != 128) || H % G || vshare < 1 || G % vshare || ld % 8 || ((uintptr_t)qkvg & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15))
    return -1;
  FastParams fp{DecodeParams{qkvg, ld, out, temp, sink, kc, vc, lens, slots, H, G, d, d, rows, window, keep, gate, do_norm, dt, scale, slope_base, eps, vshare, dt},
                part_acc, part_ml, splits};
  if (dt == 1) return d == 128 ? launch_fast<__nv_bfloat16, 128>(fp, B, s) : launch_fast<__nv_bfloat16, 64>(fp, B, s);
  return d == 128 ? launch_fast<__half, 128>(fp, B, s) : launch_fast<__half, 64>(fp, B, s);
}

extern "C" int rb_qk_head_norm(void* x, int64_t ld, int dt, const void* wq, const void* wk, int64_t T, int nq, int nk, int d, float eps,
                               cudaStream_t s) {
  const int64_t n = T * (nq + nk);
  if (n == 0) return 0;
  return rb::launch_pdl(qk_head_norm_kernel, dim3((unsigned)RB_CEIL_DIV(n, (int64_t)4)), dim3(128), 0, s, x, ld, dt, wq, wk, T, nq, nk, d, eps) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_diff_combine(const void* a, int dta, const float* lam, void* out, int dto, int64_t T, int H, int G, int dv, float diff, float eps,
                               cudaStream_t s) {
  const int64_t n = T * H;
  if (n == 0) return 0;
  if (H % G) return -1;
  return rb::launch_pdl(diff_combine_kernel, dim3((unsigned)RB_CEIL_DIV(n, (int64_t)4)), dim3(128), 0, s, a, dta, lam, out, dto, T, H, G, dv, diff, eps) == cudaSuccess ? 0 : 2;
}
