// torch.ops.realhf_b200.* registrations of the heterogeneous-stack mechanisms (seqmix.cu, latent_attn.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

using at::Tensor;
using OptT = c10::optional<Tensor>;

#define CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
#define CHECK_IN(x) \
  CHECK_CUDA(x);    \
  TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static inline int dt_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
static inline const int* int_ptr(const OptT& t, int64_t n, const char* what) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kInt && t->numel() >= n, what, ": int32 CUDA tensor expected");
  return t->data_ptr<int>();
}

extern "C" {
int rb_sublayer_input(const void*, int, const void*, const void*, int, void*, int, const int*, float*, const int*, const int*, int64_t, int,
                      int, int, float, cudaStream_t);
int rb_sublayer_input_step(const void*, int, const void*, const void*, int, void*, int, float*, const int*, int64_t, int, int, int, float,
                           cudaStream_t);
int rb_residual_add_norm(void*, int, const void*, int, const void*, int, int64_t, int, int, float, cudaStream_t);
int rb_clamped_glu(const void*, void*, int, int64_t, int, float, float, cudaStream_t);
int rb_softcap(const void*, int, float*, int64_t, float, cudaStream_t);
int rb_latent_norm_store(const void*, int64_t, int, const void*, void*, void*, const int*, const int*, const int*, int64_t, int, int, float,
                         int, cudaStream_t);
int rb_latent_window_attention(const void*, int64_t, const void*, int64_t, const int*, void*, int64_t, int, int, int, float, int, int,
                               cudaStream_t);
int rb_latent_decode_attention(const void*, int64_t, const void*, const void*, void*, const int*, const int*, void*, int, int, int, int, int,
                               int, float, int, float, int, cudaStream_t);
int rb_latent_append(const void*, int64_t, int, const void*, void*, const int*, const int*, int, int, int, float, int, cudaStream_t);
int rb_latent_decode_core(const float*, const void*, const int*, const int*, float*, float*, float*, int, int, int, int, int, int, int, const float*,
                          cudaStream_t);
}

namespace {

// state: [n_slots, taps - 1, W] fp32 or absent
void sublayer_input(const Tensor& x, const Tensor& w, const OptT& conv_w, const OptT& pos, Tensor out, const OptT& state, const OptT& tok_slot,
                    const OptT& remain, int64_t groups, double eps) {
  CHECK_IN(x); CHECK_IN(w); CHECK_IN(out);
  const int W = x.size(-1);
  const int64_t rows = x.numel() / W;
  TORCH_CHECK(w.numel() == W && out.numel() == x.numel());
  int taps = 0;
  const void* cw = nullptr;
  if (conv_w.has_value()) {
    CHECK_IN((*conv_w));
    TORCH_CHECK(conv_w->dim() == 2 && conv_w->size(1) == W && conv_w->scalar_type() == w.scalar_type(), "conv_w: tap-major [taps, W]");
    taps = conv_w->size(0);
    cw = conv_w->data_ptr();
    TORCH_CHECK(taps <= 1 || pos.has_value(), "a convolution over time needs the tokens' positions");
  }
  float* st = nullptr;
  if (state.has_value() && taps > 1) {
    CHECK_IN((*state));
    TORCH_CHECK(state->scalar_type() == at::kFloat && state->dim() == 3 && state->size(1) == taps - 1 && state->size(2) == W);
    TORCH_CHECK(tok_slot.has_value() && remain.has_value());
    st = state->data_ptr<float>();
  }
  c10::cuda::CUDAGuard g(x.device());
  const int rc = rb_sublayer_input(x.data_ptr(), dt_code(x), w.data_ptr(), cw, dt_code(w), out.data_ptr(), dt_code(out),
                                   int_ptr(pos, rows, "pos"), st, st ? int_ptr(tok_slot, rows, "tok_slot") : nullptr,
                                   st ? int_ptr(remain, rows, "remain") : nullptr, rows, W, (int)groups, taps, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "sublayer_input: unsupported shape (rc ", rc, ")");
}

void sublayer_input_step(const Tensor& x, const Tensor& w, const OptT& conv_w, Tensor out, const OptT& state, const OptT& slots, int64_t groups,
                         double eps) {
  CHECK_IN(x); CHECK_IN(w); CHECK_IN(out);
  const int W = x.size(-1);
  const int64_t rows = x.numel() / W;
  int taps = 0;
  const void* cw = nullptr;
  float* st = nullptr;
  if (conv_w.has_value()) {
    CHECK_IN((*conv_w));
    TORCH_CHECK(conv_w->dim() == 2 && conv_w->size(1) == W && conv_w->scalar_type() == w.scalar_type(), "conv_w: tap-major [taps, W]");
    taps = conv_w->size(0);
    cw = conv_w->data_ptr();
    if (taps > 1) {
      TORCH_CHECK(state.has_value(), "a convolution over time needs its state");
      CHECK_IN((*state));
      TORCH_CHECK(state->scalar_type() == at::kFloat && state->dim() == 3 && state->size(1) == taps - 1 && state->size(2) == W);
      TORCH_CHECK(slots.has_value() || state->size(0) >= rows);
      st = state->data_ptr<float>();
    }
  }
  c10::cuda::CUDAGuard g(x.device());
  const int rc = rb_sublayer_input_step(x.data_ptr(), dt_code(x), w.data_ptr(), cw, dt_code(w), out.data_ptr(), dt_code(out), st,
                                        int_ptr(slots, rows, "slots"), rows, W, (int)groups, taps, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "sublayer_input_step: unsupported shape (rc ", rc, ")");
}

void residual_add_norm_(Tensor x, const Tensor& y, const OptT& w, int64_t groups, double eps) {
  CHECK_IN(x); CHECK_IN(y);
  const int W = x.size(-1);
  TORCH_CHECK(y.numel() == x.numel());
  if (w.has_value()) { CHECK_IN((*w)); TORCH_CHECK(w->numel() == W); }
  c10::cuda::CUDAGuard g(x.device());
  const int rc = rb_residual_add_norm(x.data_ptr(), dt_code(x), y.data_ptr(), dt_code(y), w.has_value() ? w->data_ptr() : nullptr,
                                      w.has_value() ? dt_code(*w) : 0, x.numel() / W, W, (int)groups, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "residual_add_norm_: unsupported shape (rc ", rc, ")");
}

Tensor clamped_glu(const Tensor& gu, double limit, double alpha) {
  CHECK_IN(gu);
  const int F = gu.size(-1) / 2;
  auto sizes = gu.sizes().vec();
  sizes.back() = F;
  c10::cuda::CUDAGuard g(gu.device());
  auto out = at::empty(sizes, gu.options());
  TORCH_CHECK(rb_clamped_glu(gu.data_ptr(), out.data_ptr(), dt_code(gu), F ? gu.numel() / (2 * F) : 0, F, (float)limit, (float)alpha, cur_stream()) == 0);
  return out;
}

Tensor softcap(const Tensor& x, double cap) {
  CHECK_IN(x);
  c10::cuda::CUDAGuard g(x.device());
  auto out = at::empty(x.sizes(), x.options().dtype(at::kFloat));
  TORCH_CHECK(rb_softcap(x.data_ptr(), dt_code(x), out.data_ptr<float>(), x.numel(), (float)cap, cur_stream()) == 0);
  return out;
}

// qc [T, ld] (row stride ld, unit column stride); the latent occupies columns [n_q, n_q + rank), rank = w_ln.numel()
Tensor latent_norm_store(const Tensor& qc, int64_t n_q, const Tensor& w_ln, double eps, const OptT& cache, const OptT& tok_slot, const Tensor& pos,
                         const OptT& remain) {
  CHECK_CUDA(qc); CHECK_IN(w_ln);
  TORCH_CHECK(qc.dim() == 2 && qc.stride(1) == 1 && w_ln.scalar_type() == qc.scalar_type());
  const int rank = w_ln.numel();
  const int64_t T = qc.size(0);
  TORCH_CHECK(qc.size(1) >= n_q + rank);
  c10::cuda::CUDAGuard g(qc.device());
  auto c = at::empty({T, rank}, qc.options());
  void* cp = nullptr;
  int R = 1;
  if (cache.has_value()) {
    CHECK_IN((*cache));
    TORCH_CHECK(cache->dim() == 3 && cache->size(2) == rank && cache->scalar_type() == qc.scalar_type() && tok_slot.has_value() && remain.has_value());
    cp = cache->data_ptr();
    R = cache->size(1);
  }
  const int rc = rb_latent_norm_store(qc.data_ptr(), qc.stride(0), (int)n_q, w_ln.data_ptr(), c.data_ptr(), cp,
                                      cp ? int_ptr(tok_slot, T, "tok_slot") : nullptr, int_ptr(pos, T, "pos"),
                                      cp ? int_ptr(remain, T, "remain") : nullptr, T, rank, R, (float)eps, dt_code(qc), cur_stream());
  TORCH_CHECK(rc == 0, "latent_norm_store failed (rc ", rc, ")");
  return c;
}

Tensor latent_window_attention(const Tensor& q, const Tensor& kv, const Tensor& pos, int64_t H, int64_t qk, int64_t vd, double scale, int64_t window) {
  CHECK_CUDA(q); CHECK_CUDA(kv);
  TORCH_CHECK(q.dim() == 2 && kv.dim() == 2 && q.stride(1) == 1 && kv.stride(1) == 1 && q.scalar_type() == kv.scalar_type());
  TORCH_CHECK(q.size(1) >= H * qk && kv.size(1) == H * (qk + vd) && kv.size(0) == q.size(0));
  const int64_t T = q.size(0);
  c10::cuda::CUDAGuard g(q.device());
  auto out = at::empty({T, H * vd}, q.options());
  const int rc = rb_latent_window_attention(q.data_ptr(), q.stride(0), kv.data_ptr(), kv.stride(0), int_ptr(pos, T, "pos"), out.data_ptr(), T, (int)H,
                                            (int)qk, (int)vd, (float)scale, (int)window, dt_code(q), cur_stream());
  TORCH_CHECK(rc == 0, "latent_window_attention: unsupported shape (rc ", rc, ")");
  return out;
}

Tensor latent_decode_attention(const Tensor& qc, const OptT& w_ln, const Tensor& w_ukv, Tensor cache, const Tensor& cache_lens, const OptT& slots,
                               int64_t H, int64_t qk, int64_t vd, double scale, int64_t window, double eps) {
  CHECK_CUDA(qc); CHECK_IN(w_ukv); CHECK_IN(cache); CHECK_IN(cache_lens);
  TORCH_CHECK(qc.dim() == 2 && qc.stride(1) == 1 && cache.dim() == 3 && cache_lens.scalar_type() == at::kInt);
  const int rank = cache.size(2);
  const int64_t B = qc.size(0);
  TORCH_CHECK(w_ukv.dim() == 2 && w_ukv.size(0) == H * (qk + vd) && w_ukv.size(1) == rank);
  TORCH_CHECK(w_ukv.scalar_type() == qc.scalar_type() && cache.scalar_type() == qc.scalar_type());
  TORCH_CHECK(qc.size(1) >= H * qk + (w_ln.has_value() ? rank : 0));
  TORCH_CHECK(slots.has_value() || cache.size(0) >= B);
  if (w_ln.has_value()) { CHECK_IN((*w_ln)); TORCH_CHECK(w_ln->numel() == rank && w_ln->scalar_type() == qc.scalar_type()); }
  c10::cuda::CUDAGuard g(qc.device());
  auto out = at::empty({B, H * vd}, qc.options());
  const int rc = rb_latent_decode_attention(qc.data_ptr(), qc.stride(0), w_ln.has_value() ? w_ln->data_ptr() : nullptr, w_ukv.data_ptr(),
                                            cache.data_ptr(), cache_lens.data_ptr<int>(), int_ptr(slots, B, "slots"), out.data_ptr(), (int)B, (int)H,
                                            (int)qk, (int)vd, rank, (int)cache.size(1), (float)scale, (int)window, (float)eps, dt_code(qc),
                                            cur_stream());
  TORCH_CHECK(rc == 0, "latent_decode_attention: unsupported shape (rc ", rc, ")");
  return out;
}

// Normalise the latent columns of qc [B, >= n_q + rank] and append them to the ring cache at position cache_lens[slot].
void latent_append(const Tensor& qc, int64_t n_q, const Tensor& w_ln, Tensor cache, const Tensor& cache_lens, const OptT& slots, double eps) {
  CHECK_CUDA(qc); CHECK_IN(w_ln); CHECK_IN(cache); CHECK_IN(cache_lens);
  const int rank = cache.size(2);
  const int64_t B = qc.size(0);
  TORCH_CHECK(qc.dim() == 2 && qc.stride(1) == 1 && qc.size(1) >= n_q + rank && w_ln.numel() == rank && cache.dim() == 3);
  TORCH_CHECK(cache.scalar_type() == qc.scalar_type() && w_ln.scalar_type() == qc.scalar_type() && cache_lens.scalar_type() == at::kInt);
  TORCH_CHECK(slots.has_value() || cache.size(0) >= B);
  c10::cuda::CUDAGuard g(qc.device());
  const int rc = rb_latent_append(qc.data_ptr(), qc.stride(0), (int)n_q, w_ln.data_ptr(), cache.data_ptr(), cache_lens.data_ptr<int>(),
                                  int_ptr(slots, B, "slots"), (int)B, rank, (int)cache.size(1), (float)eps, dt_code(qc), cur_stream());
  TORCH_CHECK(rc == 0, "latent_append failed (rc ", rc, ")");
}

// qa [H, B, rank] fp32 (queries in latent space, scale applied) -> softmax-weighted sums of the cached latents [H, B, rank] fp32.
Tensor latent_decode_core(const Tensor& qa, const Tensor& cache, const Tensor& cache_lens, const OptT& slots, int64_t window, int64_t splits,
                         const OptT& sink) {
  CHECK_IN(qa); CHECK_IN(cache); CHECK_IN(cache_lens);
  TORCH_CHECK(qa.dim() == 3 && qa.scalar_type() == at::kFloat && cache.dim() == 3 && cache.size(2) == qa.size(2));
  TORCH_CHECK(cache_lens.scalar_type() == at::kInt);
  const int64_t H = qa.size(0), B = qa.size(1), rank = qa.size(2);
  TORCH_CHECK(slots.has_value() || cache.size(0) >= B);
  if (sink.has_value()) TORCH_CHECK(sink->is_cuda() && sink->is_contiguous() && sink->scalar_type() == at::kFloat && sink->numel() == H, "sink: fp32 [H]");
  c10::cuda::CUDAGuard g(qa.device());
  auto out = at::empty_like(qa);
  Tensor pa, pm;
  if (splits > 1) {
    pa = at::empty({H, B, splits, rank}, qa.options());
    pm = at::empty({H, B, splits, 2}, qa.options());
  }
  const int rc = rb_latent_decode_core(qa.data_ptr<float>(), cache.data_ptr(), cache_lens.data_ptr<int>(), int_ptr(slots, B, "slots"),
                                       out.data_ptr<float>(), splits > 1 ? pa.data_ptr<float>() : nullptr,
                                       splits > 1 ? pm.data_ptr<float>() : nullptr, (int)B, (int)H, (int)rank, (int)cache.size(1), (int)window,
                                       (int)splits, dt_code(cache), sink.has_value() ? sink->data_ptr<float>() : nullptr, cur_stream());
  TORCH_CHECK(rc == 0, "latent_decode_core: unsupported shape (rc ", rc, ")");
  return out;
}

}  // namespace

void register_seq_ops(torch::Library& m) {
  m.def("sublayer_input(Tensor x, Tensor w, Tensor? conv_w, Tensor? pos, Tensor(a!) out, Tensor(b!)? state, Tensor? tok_slot, Tensor? remain, int groups, float eps) -> ()", &sublayer_input);
  m.def("sublayer_input_step(Tensor x, Tensor w, Tensor? conv_w, Tensor(a!) out, Tensor(b!)? state, Tensor? slots, int groups, float eps) -> ()", &sublayer_input_step);
  m.def("residual_add_norm_(Tensor(a!) x, Tensor y, Tensor? w, int groups, float eps) -> ()", &residual_add_norm_);
  m.def("clamped_glu(Tensor gu, float limit, float alpha) -> Tensor", &clamped_glu);
  m.def("softcap(Tensor x, float cap) -> Tensor", &softcap);
  m.def("latent_norm_store(Tensor qc, int n_q, Tensor w_ln, float eps, Tensor(a!)? cache, Tensor? tok_slot, Tensor pos, Tensor? remain) -> Tensor", &latent_norm_store);
  m.def("latent_window_attention(Tensor q, Tensor kv, Tensor pos, int n_heads, int qk, int vd, float scale, int window) -> Tensor", &latent_window_attention);
  m.def("latent_append(Tensor qc, int n_q, Tensor w_ln, Tensor(a!) cache, Tensor cache_lens, Tensor? slots, float eps) -> ()", &latent_append);
  m.def("latent_decode_core(Tensor qa, Tensor cache, Tensor cache_lens, Tensor? slots, int window, int splits, Tensor? sink=None) -> Tensor", &latent_decode_core);
  m.def("latent_decode_attention(Tensor qc, Tensor? w_ln, Tensor w_ukv, Tensor(a!) cache, Tensor cache_lens, Tensor? slots, int n_heads, int qk, int vd, float scale, int window, float eps) -> Tensor", &latent_decode_attention);
}
