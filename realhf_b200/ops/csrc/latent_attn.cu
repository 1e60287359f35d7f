// Latent attention: keys and values are up-projections of one cached low-rank latent per token; no positional rotation; an
// optional sliding window (a query at position i sees positions (i - window, i]).
//
//   latent_norm_store        packed prefill: c = RMSNorm(latent part of the fused q|latent projection) * w, written packed
//                            [T, rank] (input of the key/value up-projection GEMM) and into the ring cache of its sequence
//   latent_window_attention  packed prefill over the up-projected keys / values: 16 queries x 1 head per CTA, key tiles staged
//                            in shared memory, online softmax
//   decode (one token per row; keys / values are never formed: the query is multiplied into the latent space, q W_uk, scores and
//   the weighted sum run over the cached latents, W_uv is applied to the result)
//     split form (default): latent_append + latent_decode_core (+ latent_decode_combine); the two small per-head projections
//                            are batched matrix products issued by the caller
//     latent_decode_attention  the whole step in one launch per (row, head), a block that owns its latent also normalises
//                            and appends the new row: small problems and A/B runs (`REAL_LATENT_DECODE=fused`)
//
// Scores, softmax and all accumulations are fp32; storage is T (bf16 / fp16 / fp32).  Compiled without fast-math.
// The cache of a slot is a ring of R rows: position p lives in row p % R.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------ latent_norm_store
template <typename T>
__global__ void __launch_bounds__(128) latent_norm_store_kernel(const T* __restrict__ qc, int64_t ldq, int n_q, const T* __restrict__ w,
                                                                T* __restrict__ c_out, T* __restrict__ cache, const int* __restrict__ tok_slot,
                                                                const int* __restrict__ pos, const int* __restrict__ remain, int64_t n_tok,
                                                                int rank, int R, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tok) return;
  const T* src = qc + t * ldq + n_q;
  float s = 0.f;
  for (int r = lane; r < rank; r += 32) { const float v = rb::to_f(src[r]); s += v * v; }
  s = rb::warp_sum(s);
  const float rstd = 1.f / sqrtf(s / (float)rank + eps);
  // only the last R tokens of a sequence go to its ring: earlier ones would land in rows that later positions own
  const int slot = (cache != nullptr && tok_slot != nullptr && remain[t] < R) ? tok_slot[t] : -1;
  T* dst = slot >= 0 ? cache + ((int64_t)slot * R + (pos[t] % R)) * rank : nullptr;
  for (int r = lane; r < rank; r += 32) {
    const T v = rb::from_f<T>(rb::to_f(src[r]) * rstd * rb::to_f(w[r]));
    c_out[t * rank + r] = v;
    if (dst != nullptr) dst[r] = v;
  }
}

// ------------------------------------------------------------------------------------------------ prefill
constexpr int kBQ = 16;    // queries per CTA
constexpr int kBK = 32;    // keys per shared-memory tile
constexpr int kPT = 128;   // threads: 8 per query

// Thread (i = tid / 8, c = tid % 8) owns query i's scores of keys c, c + 8, c + 16, c + 24 of a tile and its output columns
// c, c + 8, ...  NACC = ceil(vd / 8) accumulators per thread.
template <typename T, int NACC>
__global__ void __launch_bounds__(kPT) latent_window_attention_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ kv, int64_t ldkv,
                                                                      const int* __restrict__ pos, T* __restrict__ out, int64_t n_tok, int H,
                                                                      int qk, int vd, float scale, int window) {
  extern __shared__ float sm[];
  float* qs = sm;                          // [kBQ][qk]
  float* ks = qs + kBQ * qk;               // [kBK][qk + 1]
  float* vs = ks + kBK * (qk + 1);         // [kBK][vd]
  float* ps = vs + kBK * vd;               // [kBQ][kBK]
  __shared__ int64_t lo_s[kBQ];
  const int tid = threadIdx.x, i = tid >> 3, c = tid & 7;
  const int h = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kBQ;
  const int nq_valid = (int)min((int64_t)kBQ, n_tok - t0);
  if (tid < kBQ) {
    int64_t lo = INT64_MAX;
    if (tid < nq_valid) {
      const int p = pos[t0 + tid];
      const int reach = (window > 0 && window - 1 < p) ? window - 1 : p;
      lo = t0 + tid - reach;
    }
    lo_s[tid] = lo;
  }
  for (int e = tid; e < kBQ * qk; e += kPT) {
    const int r = e / qk, d = e % qk;
    qs[e] = r < nq_valid ? rb::to_f(q[(t0 + r) * ldq + (int64_t)h * qk + d]) : 0.f;
  }
  __syncthreads();
  int64_t tile_lo = INT64_MAX;
  for (int r = 0; r < nq_valid; ++r) tile_lo = min(tile_lo, lo_s[r]);
  const int64_t tile_hi = t0 + nq_valid - 1;
  const bool q_ok = i < nq_valid;
  const int64_t my_t = t0 + i, my_lo = q_ok ? lo_s[i] : INT64_MAX;
  float m = -INFINITY, l = 0.f, acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  const int64_t k_off = (int64_t)h * qk, v_off = (int64_t)H * qk + (int64_t)h * vd;
  for (int64_t kb = tile_lo; kb <= tile_hi; kb += kBK) {
    const int nk = (int)min((int64_t)kBK, tile_hi - kb + 1);
    for (int e = tid; e < kBK * qk; e += kPT) {
      const int r = e / qk, d = e % qk;
      ks[r * (qk + 1) + d] = r < nk ? rb::to_f(kv[(kb + r) * ldkv + k_off + d]) : 0.f;
    }
    for (int e = tid; e < kBK * vd; e += kPT) {
      const int r = e / vd, d = e % vd;
      vs[e] = r < nk ? rb::to_f(kv[(kb + r) * ldkv + v_off + d]) : 0.f;
    }
    __syncthreads();
    float sc[kBK / 8];
    float cmax = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < kBK / 8; ++jj) {
      const int j = c + 8 * jj;
      const int64_t key = kb + j;
      float s = -INFINITY;
      if (q_ok && j < nk && key >= my_lo && key <= my_t) {
        float d_ = 0.f;
        const float* qr = qs + i * qk;
        const float* kr = ks + j * (qk + 1);
        for (int d = 0; d < qk; ++d) d_ = fmaf(qr[d], kr[d], d_);
        s = d_ * scale;
      }
      sc[jj] = s;
      cmax = fmaxf(cmax, s);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
    const float m_new = fmaxf(m, cmax);
    float corr = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {                      // no visible key so far: nothing to add
#pragma unroll
      for (int jj = 0; jj < kBK / 8; ++jj) ps[i * kBK + c + 8 * jj] = 0.f;
    } else {
      corr = expf(m - m_new);                      // m = -inf: 0
#pragma unroll
      for (int jj = 0; jj < kBK / 8; ++jj) {
        const float p = expf(sc[jj] - m_new);      // masked: exp(-inf) = 0
        ps[i * kBK + c + 8 * jj] = p;
        psum += p;
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * corr + psum;
    m = m_new;
    __syncthreads();
    const float* pr = ps + i * kBK;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int e = c + 8 * a;
      float v = acc[a] * corr;
      if (e < vd)
        for (int j = 0; j < nk; ++j) v = fmaf(pr[j], vs[j * vd + e], v);
      acc[a] = v;
    }
    __syncthreads();
  }
  if (q_ok) {
    const float inv = 1.f / l;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int e = c + 8 * a;
      if (e < vd) out[my_t * ((int64_t)H * vd) + (int64_t)h * vd + e] = rb::from_f<T>(acc[a] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int kDT = 128;         // threads per (row, head) CTA
constexpr int kMaxRankRegs = 16; // latent rank <= 32 * 16 = 512

template <typename T>
__global__ void __launch_bounds__(kDT) latent_decode_attention_kernel(
    const T* __restrict__ qc, int64_t ldq, const T* __restrict__ w_ln, const T* __restrict__ w_ukv, T* __restrict__ cache,
    const int* __restrict__ cache_lens, const int* __restrict__ slots, T* __restrict__ out, int H, int qk, int vd, int rank, int R,
    float scale, int window, float eps) {
  extern __shared__ float sm[];
  float* qa = sm;                    // [rank]  query in latent space, times scale
  float* cnew = qa + rank;           // [rank]  this token's latent (own-latent blocks)
  float* accw = cnew + rank;         // [nwarp][rank]
  float* qsm = accw + (kDT / 32) * rank;  // [qk]
  __shared__ float red[32];
  __shared__ float mw[kDT / 32], lw[kDT / 32];
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t slot = slots != nullptr ? slots[b] : b;
  const int pos = cache_lens[slot];
  const int n_q = H * qk;
  const bool own = w_ln != nullptr;
  T* crow_new = cache + (slot * R + (pos % R)) * (int64_t)rank;
  if (own) {
    float s = 0.f;
    for (int r = tid; r < rank; r += kDT) { const float v = rb::to_f(qc[b * ldq + n_q + r]); s += v * v; }
    s = rb::block_reduce<false>(s, red);
    const float rstd = 1.f / sqrtf(s / (float)rank + eps);
    for (int r = tid; r < rank; r += kDT) {
      const T v = rb::from_f<T>(rb::to_f(qc[b * ldq + n_q + r]) * rstd * rb::to_f(w_ln[r]));
      cnew[r] = rb::to_f(v);
      if (h == 0) crow_new[r] = v;
    }
  }
  for (int d = tid; d < qk; d += kDT) qsm[d] = rb::to_f(qc[b * ldq + (int64_t)h * qk + d]);
  __syncthreads();
  for (int r = tid; r < rank; r += kDT) {
    float a = 0.f;
    const T* wk = w_ukv + (int64_t)h * qk * rank + r;
    for (int d = 0; d < qk; ++d) a = fmaf(qsm[d], rb::to_f(wk[(int64_t)d * rank]), a);
    qa[r] = a * scale;
  }
  __syncthreads();
  const int reach = (window > 0 && window - 1 < pos) ? window - 1 : pos;
  const int lo = pos - reach;
  float m = -INFINITY, l = 0.f, acc[kMaxRankRegs], crow[kMaxRankRegs];
#pragma unroll
  for (int k = 0; k < kMaxRankRegs; ++k) acc[k] = 0.f;
  for (int j = lo + warp; j <= pos; j += kDT / 32) {
    const bool fresh = own && j == pos;        // the row this launch appends: other CTAs may not have written it yet
    const T* cr = cache + (slot * R + (j % R)) * (int64_t)rank;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxRankRegs; ++k) {
      const int r = lane + 32 * k;
      crow[k] = r < rank ? (fresh ? cnew[r] : rb::to_f(cr[r])) : 0.f;
      s = fmaf(crow[k], r < rank ? qa[r] : 0.f, s);
    }
    s = rb::warp_sum(s);
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new), p = expf(s - m_new);
    l = l * corr + p;
    m = m_new;
#pragma unroll
    for (int k = 0; k < kMaxRankRegs; ++k) acc[k] = fmaf(p, crow[k], acc[k] * corr);
  }
  if (lane == 0) { mw[warp] = m; lw[warp] = l; }
#pragma unroll
  for (int k = 0; k < kMaxRankRegs; ++k) {
    const int r = lane + 32 * k;
    if (r < rank) accw[warp * rank + r] = acc[k];
  }
  __syncthreads();
  float M = -INFINITY;
  for (int w_ = 0; w_ < kDT / 32; ++w_) M = fmaxf(M, mw[w_]);
  float L = 0.f;
  for (int w_ = 0; w_ < kDT / 32; ++w_) L += lw[w_] * (mw[w_] == -INFINITY ? 0.f : expf(mw[w_] - M));
  __syncthreads();
  for (int r = tid; r < rank; r += kDT) {     // merged latent-space output, reusing qa
    float o = 0.f;
    for (int w_ = 0; w_ < kDT / 32; ++w_)
      if (mw[w_] != -INFINITY) o += accw[w_ * rank + r] * expf(mw[w_] - M);
    qa[r] = o / L;
  }
  __syncthreads();
  const T* wv = w_ukv + ((int64_t)n_q + (int64_t)h * vd) * rank;
  for (int e = warp; e < vd; e += kDT / 32) {
    float a = 0.f;
    for (int r = lane; r < rank; r += 32) a = fmaf(rb::to_f(wv[(int64_t)e * rank + r]), qa[r], a);
    a = rb::warp_sum(a);
    if (lane == 0) out[(int64_t)b * H * vd + (int64_t)h * vd + e] = rb::from_f<T>(a);
  }
}


// ------------------------------------------------------------------------------------------------ decode, split form
// Three steps: `latent_append` normalises and appends the new latent rows; the caller forms qa = scale * q W_uk per head with a
// batched matrix product ([H, B, rank] fp32); `latent_decode_core` below turns (qa, cached latents) into the softmax-weighted
// latent sums [H, B, rank] fp32, to which the caller applies W_uv.
//
// Core: one CTA per (row, tile of 16 heads, key split), 128 threads.  A tile of 32 latent rows is staged in shared memory in
// the cache's own type and used twice: scores S[16 heads][32 keys] (thread = 1 key x 4 heads, the dot over the rank with 16-byte shared loads;
// the qa reads are warp broadcasts) and, after an online-softmax update per head, the weighted sum into the thread's
// 16 heads x 4 rank columns of accumulators.  With more than one split the partial (max, sum, accumulator) triples go to a
// workspace and `latent_decode_combine` merges them.
// 4 consecutive elements of a shared-memory row as fp32 (the row keeps the cache's storage type: half the bytes of an fp32
// tile for 16-bit caches, so three CTAs fit an SM)
RB_DEVICE float4 ld4s(const float* p) { return *reinterpret_cast<const float4*>(p); }
RB_DEVICE float4 ld4s(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
RB_DEVICE float4 ld4s(const __half* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

constexpr int kCT = 128;     // threads
constexpr int kHT = 16;      // heads per CTA
constexpr int kKT = 32;      // keys per tile
constexpr int kMaxRank = 512;

template <typename T>
__global__ void __launch_bounds__(128) latent_append_kernel(const T* __restrict__ qc, int64_t ldq, int n_q, const T* __restrict__ w,
                                                            T* __restrict__ cache, const int* __restrict__ cache_lens,
                                                            const int* __restrict__ slots, int B, int rank, int R, float eps) {
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= B) return;
  const int64_t slot = slots != nullptr ? slots[b] : b;
  const int pos = cache_lens[slot];
  const T* src = qc + b * ldq + n_q;
  float s = 0.f;
  for (int r = lane; r < rank; r += 32) { const float v = rb::to_f(src[r]); s += v * v; }
  s = rb::warp_sum(s);
  const float rstd = 1.f / sqrtf(s / (float)rank + eps);
  T* dst = cache + (slot * R + (pos % R)) * (int64_t)rank;
  for (int r = lane; r < rank; r += 32) dst[r] = rb::from_f<T>(rb::to_f(src[r]) * rstd * rb::to_f(w[r]));
}

template <typename T>
__global__ void __launch_bounds__(kCT) latent_decode_core_kernel(const float* __restrict__ qa, const T* __restrict__ cache,
                                                                 const int* __restrict__ cache_lens, const int* __restrict__ slots,
                                                                 float* __restrict__ out, float* __restrict__ part_acc,
                                                                 float* __restrict__ part_ml, int B, int H, int rank, int R, int window,
                                                                 int splits, const float* __restrict__ sink) {
  extern __shared__ float sm[];
  const int RP = ((rank + 3) & ~3) + 4;        // padded row: 16-byte aligned, rows 4 banks apart
  float* qs = sm;                              // [kHT][RP]
  T* cs = reinterpret_cast<T*>(qs + kHT * RP); // [kKT][RP]   latent rows as stored
  float* ps = reinterpret_cast<float*>(cs + kKT * RP);   // [kKT][kHT]  scores, then softmax weights
  float* al = ps + kKT * kHT;                  // [kHT] rescale factor of the running sums for this tile
  const int tid = threadIdx.x;
  const int b = blockIdx.x, h0 = blockIdx.y * kHT, split = blockIdx.z;
  const int nh = min(kHT, H - h0);
  const int64_t slot = slots != nullptr ? slots[b] : b;
  const int pos = cache_lens[slot];
  const int reach = (window > 0 && window - 1 < pos) ? window - 1 : pos;
  const int n_keys = reach + 1, lo = pos - reach;
  const int per = RB_CEIL_DIV(RB_CEIL_DIV(n_keys, splits), kKT) * kKT;   // keys per split, whole tiles
  const int k_begin = lo + split * per, k_end = min(pos + 1, k_begin + per);
  for (int e = tid; e < kHT * RP; e += kCT) {
    const int h = e / RP, r = e % RP;
    qs[e] = (h < nh && r < rank) ? qa[((int64_t)(h0 + h) * B + b) * rank + r] : 0.f;
  }
  const bool vec = rank % (16 / (int)sizeof(T)) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0;
  if (vec)                                     // the vector fill writes columns [0, rank) only
    for (int e = tid; e < kKT * (RP - rank); e += kCT) cs[(e / (RP - rank)) * RP + rank + e % (RP - rank)] = rb::from_f<T>(0.f);
  const int my_k = tid & 31, hg = tid >> 5;    // scores: key my_k of the tile, heads 4 hg .. 4 hg + 3
  const int r0 = tid * 4;                      // sums: rank columns r0 .. r0 + 3 of all 16 heads
  float acc[kHT][4];
#pragma unroll
  for (int h = 0; h < kHT; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;        // of head `tid` (threads 0 .. 15)
  for (int kb = k_begin; kb < k_end; kb += kKT) {
    const int nk = min(kKT, k_end - kb);
    __syncthreads();                           // previous tile fully consumed (and qs written, first time round)
    if (vec) {
      // 16-byte global loads: VPT elements per thread and step, stored as two 8-byte halves (rows are 8-byte aligned); the pad
      // columns beyond the rank stay zero from the first fill
      constexpr int VPT = 16 / sizeof(T);
      const int per_row = rank / VPT;
      for (int e = tid; e < kKT * per_row; e += kCT) {
        const int k = e / per_row, v = e - k * per_row;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (k < nk) raw = *reinterpret_cast<const uint4*>(cache + (slot * R + ((kb + k) % R)) * (int64_t)rank + v * VPT);
        uint2* dst = reinterpret_cast<uint2*>(cs + k * RP + v * VPT);
        dst[0] = make_uint2(raw.x, raw.y);
        dst[1] = make_uint2(raw.z, raw.w);
      }
    } else {
      for (int e = tid; e < kKT * RP; e += kCT) {
        const int k = e / RP, r = e % RP;
        cs[e] = (k < nk && r < rank) ? cache[(slot * R + ((kb + k) % R)) * (int64_t)rank + r] : rb::from_f<T>(0.f);
      }
    }
    __syncthreads();
    {
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
      const T* cr = cs + my_k * RP;
#pragma unroll 4
      for (int r4 = 0; r4 < (RP - 4) / 4; ++r4) {
        const float4 cv = ld4s(cr + 4 * r4);
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          const float4 qv = reinterpret_cast<const float4*>(qs + (hg * 4 + hh) * RP)[r4];
          s4[hh] = fmaf(cv.x, qv.x, fmaf(cv.y, qv.y, fmaf(cv.z, qv.z, fmaf(cv.w, qv.w, s4[hh]))));
        }
      }
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) ps[my_k * kHT + hg * 4 + hh] = my_k < nk ? s4[hh] : -INFINITY;
    }
    __syncthreads();
    if (tid < kHT) {                           // online softmax of head `tid` over this tile
      float mx = m_run;
      for (int k = 0; k < nk; ++k) mx = fmaxf(mx, ps[k * kHT + tid]);
      const float a = expf(m_run - mx);        // first tile: exp(-inf) = 0
      float sum = 0.f;
      for (int k = 0; k < kKT; ++k) {
        const float p = k < nk ? expf(ps[k * kHT + tid] - mx) : 0.f;
        ps[k * kHT + tid] = p;
        sum += p;
      }
      l_run = l_run * a + sum;
      m_run = mx;
      al[tid] = a;
    }
    __syncthreads();
    if (r0 < RP - 4) {
#pragma unroll
      for (int h = 0; h < kHT; ++h) {
        const float a = al[h];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] *= a;
      }
      for (int k = 0; k < nk; ++k) {
        const float4 cv = ld4s(cs + k * RP + r0);
        const float4* pk = reinterpret_cast<const float4*>(ps + k * kHT);
#pragma unroll
        for (int h4 = 0; h4 < kHT / 4; ++h4) {
          const float4 pv = pk[h4];
          const float pw[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
          for (int hh = 0; hh < 4; ++hh) {
            acc[h4 * 4 + hh][0] = fmaf(pw[hh], cv.x, acc[h4 * 4 + hh][0]);
            acc[h4 * 4 + hh][1] = fmaf(pw[hh], cv.y, acc[h4 * 4 + hh][1]);
            acc[h4 * 4 + hh][2] = fmaf(pw[hh], cv.z, acc[h4 * 4 + hh][2]);
            acc[h4 * 4 + hh][3] = fmaf(pw[hh], cv.w, acc[h4 * 4 + hh][3]);
          }
        }
      }
    }
  }
  __syncthreads();
  if (tid < kHT) { al[tid] = l_run; ps[tid] = m_run; }
  __syncthreads();
  if (splits == 1) {
#pragma unroll
    for (int h = 0; h < kHT; ++h) {
      if (h >= nh) break;
      // a sink logit is one more term of the denominator: no key, no value
      const float inv = 1.f / (al[h] + (sink != nullptr ? expf(sink[h0 + h] - ps[h]) : 0.f));
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (r0 + i < rank) out[((int64_t)(h0 + h) * B + b) * rank + r0 + i] = acc[h][i] * inv;
    }
  } else {
#pragma unroll
    for (int h = 0; h < kHT; ++h) {
      if (h >= nh) break;
      const int64_t row = ((int64_t)(h0 + h) * B + b) * splits + split;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (r0 + i < rank) part_acc[row * rank + r0 + i] = acc[h][i];
      if (tid == 0) { part_ml[row * 2] = ps[h]; part_ml[row * 2 + 1] = al[h]; }
    }
  }
}

// out[h, b, :] = sum_s acc_s exp(m_s - M) / sum_s l_s exp(m_s - M); a split without keys has m = -inf, l = 0.
__global__ void __launch_bounds__(128) latent_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                                    float* __restrict__ out, int rank, int splits, const float* __restrict__ sink, int B) {
  const int64_t row = blockIdx.x;      // (h, b)
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(row * splits + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = part_ml[(row * splits + s) * 2];
    if (m != -INFINITY) L += part_ml[(row * splits + s) * 2 + 1] * expf(m - M);
  }
  if (sink != nullptr) L += expf(sink[row / B] - M);
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = part_ml[(row * splits + s) * 2];
      if (m != -INFINITY) o += part_acc[(row * splits + s) * rank + r] * expf(m - M);
    }
    out[row * rank + r] = o / L;
  }
}

template <typename T, int NACC>
int launch_prefill(const void* q, int64_t ldq, const void* kv, int64_t ldkv, const int* pos, void* out, int64_t n_tok, int H, int qk, int vd,
                   float scale, int window, cudaStream_t s) {
  const size_t smem = ((size_t)kBQ * qk + (size_t)kBK * (qk + 1) + (size_t)kBK * vd + (size_t)kBQ * kBK) * sizeof(float);
  if (smem > 200 * 1024) return 1;
  auto kern = latent_window_attention_kernel<T, NACC>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  dim3 grid((unsigned)RB_CEIL_DIV(n_tok, (int64_t)kBQ), (unsigned)H);
  kern<<<grid, kPT, smem, s>>>((const T*)q, ldq, (const T*)kv, ldkv, pos, (T*)out, n_tok, H, qk, vd, scale, window);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <typename T>
int dispatch_prefill(const void* q, int64_t ldq, const void* kv, int64_t ldkv, const int* pos, void* out, int64_t n_tok, int H, int qk, int vd,
                     float scale, int window, cudaStream_t s) {
  if (vd <= 64) return launch_prefill<T, 8>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s);
  if (vd <= 128) return launch_prefill<T, 16>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s);
  if (vd <= 256) return launch_prefill<T, 32>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s);
  return 1;
}

}  // namespace

#define RB_DISPATCH_T(dt, ...)                                                      \
  switch (dt) {                                                                     \
    case 0: { using T = float; __VA_ARGS__; break; }                                \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; }                        \
    case 2: { using T = __half; __VA_ARGS__; break; }                               \
    default: return 1;                                                              \
  }

extern "C" {

int rb_latent_norm_store(const void* qc, int64_t ldq, int n_q, const void* w, void* c_out, void* cache, const int* tok_slot, const int* pos,
                         const int* remain, int64_t n_tok, int rank, int R, float eps, int dt, cudaStream_t s) {
  if (n_tok == 0) return 0;
  RB_DISPATCH_T(dt, (latent_norm_store_kernel<T><<<(unsigned)RB_CEIL_DIV(n_tok, (int64_t)4), 128, 0, s>>>(
                        (const T*)qc, ldq, n_q, (const T*)w, (T*)c_out, (T*)cache, tok_slot, pos, remain, n_tok, rank, R, eps)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_latent_window_attention(const void* q, int64_t ldq, const void* kv, int64_t ldkv, const int* pos, void* out, int64_t n_tok, int H,
                               int qk, int vd, float scale, int window, int dt, cudaStream_t s) {
  if (n_tok == 0) return 0;
  RB_DISPATCH_T(dt, return dispatch_prefill<T>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s));
  return 1;
}

int rb_latent_decode_attention(const void* qc, int64_t ldq, const void* w_ln, const void* w_ukv, void* cache, const int* cache_lens,
                               const int* slots, void* out, int B, int H, int qk, int vd, int rank, int R, float scale, int window, float eps,
                               int dt, cudaStream_t s) {
  if (B == 0) return 0;
  if (rank > 32 * kMaxRankRegs) return 1;
  const size_t smem = ((size_t)(2 + kDT / 32) * rank + qk) * sizeof(float);
  if (smem > 48 * 1024) return 1;
  dim3 grid((unsigned)B, (unsigned)H);
  RB_DISPATCH_T(dt, (latent_decode_attention_kernel<T><<<grid, kDT, smem, s>>>((const T*)qc, ldq, (const T*)w_ln, (const T*)w_ukv, (T*)cache,
                                                                                cache_lens, slots, (T*)out, H, qk, vd, rank, R, scale, window, eps)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_latent_append(const void* qc, int64_t ldq, int n_q, const void* w, void* cache, const int* cache_lens, const int* slots, int B,
                     int rank, int R, float eps, int dt, cudaStream_t s) {
  if (B == 0) return 0;
  RB_DISPATCH_T(dt, (latent_append_kernel<T><<<RB_CEIL_DIV(B, 4), 128, 0, s>>>((const T*)qc, ldq, n_q, (const T*)w, (T*)cache, cache_lens,
                                                                                  slots, B, rank, R, eps)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// qa, out: [H, B, rank] fp32; sink [H] fp32 or null (a bare logit in every head's softmax denominator).  part_acc [H, B, splits, rank], part_ml [H, B, splits, 2] (splits > 1).
int rb_latent_decode_core(const float* qa, const void* cache, const int* cache_lens, const int* slots, float* out, float* part_acc,
                          float* part_ml, int B, int H, int rank, int R, int window, int splits, int dt, const float* sink, cudaStream_t s) {
  if (B == 0) return 0;
  if (rank > kMaxRank || splits < 1 || (splits > 1 && (part_acc == nullptr || part_ml == nullptr))) return 1;
  const int RP = ((rank + 3) & ~3) + 4;
  const size_t esz = dt == 0 ? 4 : 2;
  const size_t smem = ((size_t)kHT * RP + kKT * kHT + kHT) * sizeof(float) + (size_t)kKT * RP * esz;
  dim3 grid((unsigned)B, (unsigned)RB_CEIL_DIV(H, kHT), (unsigned)splits);
  RB_DISPATCH_T(dt, {
    auto kern = latent_decode_core_kernel<T>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
    kern<<<grid, kCT, smem, s>>>(qa, (const T*)cache, cache_lens, slots, out, part_acc, part_ml, B, H, rank, R, window, splits, sink);
  });
  if (cudaGetLastError() != cudaSuccess) return 2;
  if (splits > 1) {
    latent_decode_combine_kernel<<<(unsigned)(H * B), 128, 0, s>>>(part_acc, part_ml, out, rank, splits, sink, B);
    if (cudaGetLastError() != cudaSuccess) return 2;
  }
  return 0;
}

}  // extern "C"
