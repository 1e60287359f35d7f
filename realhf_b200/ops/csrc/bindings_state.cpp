// torch.ops.realhf_b200.* registrations of window attention with a sink (sinkattn.cu), the gated delta rule (delta.cu) and the
// sinusoidal embedding / concat / relu^2 row kernels (posenc.cu).
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
#define CHECK_ROWS(x) \
  CHECK_CUDA(x);      \
  TORCH_CHECK((x).dim() == 2 && (x).stride(1) == 1, #x " must be 2-D with unit column stride")

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
static inline const void* same_type_ptr(const OptT& t, const Tensor& like, int64_t n, const char* what) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == like.scalar_type() && t->numel() == n, what, ": wrong type or size");
  return t->data_ptr();
}

extern "C" {
int rb_embed_sinusoid(const int64_t*, const void*, int, const int*, const int*, const float*, float*, int64_t, int, int, cudaStream_t);
int rb_concat_cast(const void*, int, int, const void*, int, int, void*, int, int64_t, cudaStream_t);
int rb_relu2(const void*, void*, int, int64_t, cudaStream_t);
int rb_rms_norm_rows(void*, int, const void*, int, const void*, int, void*, int, int64_t, int, float, float, cudaStream_t);
int rb_value_norm_store(const void*, int64_t, int, void*, void*, void*, const int*, const int*, const int*, int64_t, int, int, int, int, int, int, int,
                        float, int, cudaStream_t);
int rb_sink_window_prefill(const void*, int64_t, const void*, void*, const void*, const void*, const int*, int, int, int, int, int, int, float, int,
                           int, float, int, int, int, int64_t, int, cudaStream_t);
int rb_sink_window_decode(const void*, int64_t, void*, const void*, const void*, void*, void*, const int*, const int*, int, int, int, int, int, int,
                          float, int, int, float, int, int, float, int, int, int, cudaStream_t);
int rb_sink_window_decode_fast(const void*, int64_t, void*, const void*, const void*, void*, void*, const int*, const int*, float*, float*, int, int,
                               int, int, int, int, float, int, int, float, int, int, float, int, int, cudaStream_t);
int rb_attn_fwd_sink(const void*, const void*, const void*, void*, const int*, int64_t, int64_t, int64_t, int64_t, int, int, int, int, int, int, float,
                     int, int, const void*, const void*, const void*, int64_t, float, int, int, cudaStream_t);
int rb_delta_prepare(const void*, int64_t, int, const void*, const void*, const void*, float*, const int*, float*, const int*, const int*, const int*,
                     int64_t, int, int, int, int, int, float, cudaStream_t);
int rb_delta_rule(const float*, float*, const int*, float*, const int*, int, int, int, int, int, int, cudaStream_t);
int rb_gated_head_norm(const float*, const void*, int, const void*, int64_t, int, void*, int, int64_t, int, int, float, cudaStream_t);
}

namespace {

void embed_sinusoid(const Tensor& ids, const Tensor& wte, const Tensor& pos, const OptT& slots, const Tensor& inv_freq, Tensor out) {
  CHECK_IN(ids); CHECK_IN(wte); CHECK_IN(pos); CHECK_IN(inv_freq); CHECK_IN(out);
  const int64_t T = ids.numel();
  const int W = wte.size(1);
  TORCH_CHECK(ids.scalar_type() == at::kLong && pos.scalar_type() == at::kInt && inv_freq.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat);
  TORCH_CHECK(out.numel() == T * W && inv_freq.numel() >= (W + 1) / 2 && (slots.has_value() || pos.numel() >= T));
  c10::cuda::CUDAGuard g(wte.device());
  TORCH_CHECK(rb_embed_sinusoid(ids.data_ptr<int64_t>(), wte.data_ptr(), dt_code(wte), pos.data_ptr<int>(), int_ptr(slots, T, "slots"),
                                inv_freq.data_ptr<float>(), out.data_ptr<float>(), T, W, (int)wte.size(0), cur_stream()) == 0);
}

void concat_cast(const Tensor& a, const Tensor& b, Tensor out) {
  CHECK_IN(a); CHECK_IN(b); CHECK_IN(out);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(0) == b.size(0) && out.numel() == a.numel() + b.numel());
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(rb_concat_cast(a.data_ptr(), dt_code(a), (int)a.size(1), b.data_ptr(), dt_code(b), (int)b.size(1), out.data_ptr(), dt_code(out),
                             a.size(0), cur_stream()) == 0);
}

Tensor relu2(const Tensor& x) {
  CHECK_IN(x);
  c10::cuda::CUDAGuard g(x.device());
  auto out = at::empty_like(x);
  TORCH_CHECK(rb_relu2(x.data_ptr(), out.data_ptr(), dt_code(x), x.numel(), cur_stream()) == 0);
  return out;
}

// out = rmsnorm(x) * (w + w_offset); with y: x += y in place first
void rms_norm_rows(Tensor x, const OptT& y, const Tensor& w, Tensor out, double eps, double w_offset) {
  CHECK_IN(x); CHECK_IN(w); CHECK_IN(out);
  const int W = x.size(-1);
  TORCH_CHECK(w.numel() == W && out.numel() == x.numel());
  if (y.has_value()) { CHECK_IN((*y)); TORCH_CHECK(y->numel() == x.numel()); }
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(rb_rms_norm_rows(x.data_ptr(), dt_code(x), y.has_value() ? y->data_ptr() : nullptr, y.has_value() ? dt_code(*y) : 0, w.data_ptr(),
                               dt_code(w), out.data_ptr(), dt_code(out), x.numel() / W, W, (float)eps, (float)w_offset, cur_stream()) == 0);
}

// caches: kc [n_slots, G, rows, d], vc [n_slots, G / vshare, rows, dv] (vshare consecutive key heads read one value head)
void value_norm_store(const Tensor& qkvg, Tensor vout, const OptT& kc, const OptT& vc, const OptT& tok_slot, const Tensor& pos, const OptT& remain,
                      int64_t H, int64_t G, int64_t d, int64_t dv, int64_t keep, bool do_norm, double eps, int64_t vshare) {
  CHECK_ROWS(qkvg); CHECK_IN(vout);
  const int64_t T = qkvg.size(0);
  TORCH_CHECK(vshare >= 1 && G % vshare == 0);
  const int64_t Gv = G / vshare;
  TORCH_CHECK(qkvg.size(1) >= H * d + G * d + Gv * dv && vout.numel() == T * Gv * dv && vout.scalar_type() == qkvg.scalar_type());
  int rows = 1;
  void *kp = nullptr, *vp = nullptr;
  if (kc.has_value()) {
    CHECK_IN((*kc)); CHECK_IN((*vc));
    TORCH_CHECK(kc->dim() == 4 && kc->size(1) == G && kc->size(3) == d && vc->size(1) == Gv && vc->size(3) == dv && vc->size(2) == kc->size(2));
    TORCH_CHECK(kc->scalar_type() == qkvg.scalar_type() && vc->scalar_type() == qkvg.scalar_type() && tok_slot.has_value() && remain.has_value());
    rows = kc->size(2); kp = kc->data_ptr(); vp = vc->data_ptr();
  }
  c10::cuda::CUDAGuard g(qkvg.device());
  TORCH_CHECK(rb_value_norm_store(qkvg.data_ptr(), qkvg.stride(0), dt_code(qkvg), vout.data_ptr(), kp, vp, kp ? int_ptr(tok_slot, T, "tok_slot") : nullptr,
                                  int_ptr(pos, T, "pos"), kp ? int_ptr(remain, T, "remain") : nullptr, T, (int)H, (int)G, (int)d, (int)dv, (int)keep, rows,
                                  do_norm ? 1 : 0, (float)eps, (int)vshare, cur_stream()) == 0);
}

void sink_window_attention(const Tensor& qkvg, const Tensor& vn, Tensor out, const OptT& temp, const OptT& sink, const Tensor& cu, int64_t max_seqlen,
                           int64_t H, int64_t G, int64_t d, int64_t dv, double scale, int64_t window, int64_t keep, double slope_base, bool gate,
                           int64_t vshare) {
  // vn: rows of G / vshare value heads (any row stride); out in its own type (fp32 keeps the weighted sums unrounded)
  CHECK_ROWS(qkvg); CHECK_ROWS(vn); CHECK_IN(out); CHECK_IN(cu);
  const int64_t T = qkvg.size(0);
  TORCH_CHECK(vshare >= 1 && G % vshare == 0);
  TORCH_CHECK(qkvg.size(1) >= H * d + G * d + (gate ? G / vshare * dv + H : 0) && vn.size(0) == T && vn.size(1) >= G / vshare * dv && out.numel() == T * H * dv);
  TORCH_CHECK(vn.scalar_type() == qkvg.scalar_type() && cu.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard g(qkvg.device());
  const int rc = rb_sink_window_prefill(qkvg.data_ptr(), qkvg.stride(0), vn.data_ptr(), out.data_ptr(), same_type_ptr(temp, qkvg, H, "temp"),
                                        same_type_ptr(sink, qkvg, H, "sink"), cu.data_ptr<int>(), (int)cu.numel() - 1, (int)max_seqlen, (int)H, (int)G,
                                        (int)d, (int)dv, (float)scale, (int)window, (int)keep, (float)slope_base, gate ? 1 : 0, dt_code(qkvg), (int)vshare,
                                        vn.stride(0), dt_code(out), cur_stream());
  TORCH_CHECK(rc == 0, "sink_window_attention: unsupported shape (rc ", rc, ")");
}

// tensor-core form: 16-bit operands, equal query / value head size of 64 or 128
void sink_window_attention_tc(const Tensor& qkvg, const Tensor& vn, Tensor out, const OptT& temp, const OptT& sink, const Tensor& cu, int64_t max_seqlen,
                              int64_t H, int64_t G, int64_t d, double scale, int64_t window, int64_t keep, double slope_base, bool gate,
                              int64_t vshare) {
  CHECK_ROWS(qkvg); CHECK_ROWS(vn); CHECK_IN(out); CHECK_IN(cu);
  const int64_t T = qkvg.size(0);
  TORCH_CHECK(vshare >= 1 && G % vshare == 0);
  TORCH_CHECK(qkvg.size(1) >= H * d + G * d + (gate ? G / vshare * d + H : 0) && vn.size(0) == T && vn.size(1) >= G / vshare * d && out.numel() == T * H * d);
  TORCH_CHECK(vn.scalar_type() == qkvg.scalar_type() && out.scalar_type() == qkvg.scalar_type() && cu.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard g(qkvg.device());
  const char* base = static_cast<const char*>(qkvg.data_ptr());
  const int es = (int)qkvg.element_size();
  const int rc = rb_attn_fwd_sink(base, base + H * d * es, vn.data_ptr(), out.data_ptr(), cu.data_ptr<int>(), qkvg.stride(0), qkvg.stride(0), vn.stride(0),
                                  H * d, (int)T, (int)cu.numel() - 1, (int)H, (int)G, (int)d, (int)max_seqlen, (float)scale, (int)window, (int)keep,
                                  same_type_ptr(temp, qkvg, H, "temp"), same_type_ptr(sink, qkvg, H, "sink"),
                                  gate ? base + (H * d + G * d + G / vshare * d) * es : nullptr, qkvg.stride(0), (float)slope_base, dt_code(qkvg),
                                  (int)vshare, cur_stream());
  TORCH_CHECK(rc == 0, "sink_window_attention_tc: unsupported shape (rc ", rc, ")");
}

void sink_window_decode_attention(const Tensor& qkvg, Tensor out, const OptT& temp, const OptT& sink, Tensor kc, Tensor vc, const Tensor& lens,
                                  const OptT& slots, int64_t H, int64_t G, int64_t d, int64_t dv, double scale, int64_t window, int64_t keep,
                                  double slope_base, bool gate, bool do_norm, double eps, int64_t vshare) {
  CHECK_ROWS(qkvg); CHECK_IN(out); CHECK_IN(kc); CHECK_IN(vc); CHECK_IN(lens);
  const int64_t B = qkvg.size(0);
  TORCH_CHECK(vshare >= 1 && G % vshare == 0);
  const int64_t Gv = G / vshare;
  TORCH_CHECK(qkvg.size(1) >= H * d + G * d + Gv * dv + (gate ? H : 0) && out.numel() == B * H * dv && lens.scalar_type() == at::kInt);
  TORCH_CHECK(kc.dim() == 4 && kc.size(1) == G && kc.size(3) == d && vc.size(1) == Gv && vc.size(3) == dv && vc.size(2) == kc.size(2));
  TORCH_CHECK(kc.scalar_type() == qkvg.scalar_type() && vc.scalar_type() == qkvg.scalar_type());
  TORCH_CHECK(out.scalar_type() == qkvg.scalar_type() || out.scalar_type() == at::kFloat);
  TORCH_CHECK(slots.has_value() || kc.size(0) >= B);
  c10::cuda::CUDAGuard g(qkvg.device());
  const int rep = (int)(H / G);
  if (qkvg.scalar_type() != at::kFloat && out.scalar_type() == qkvg.scalar_type() && d == dv && (d == 64 || d == 128) && (rep == 1 || rep == 2 || rep == 4 || rep == 8) &&
      qkvg.stride(0) % 8 == 0 && (H * d) % 8 == 0 && reinterpret_cast<uintptr_t>(qkvg.data_ptr()) % 16 == 0) {
    // enough CTAs for two per SM, at least 128 keys per split (the cache's row count bounds the visible keys).  Measured at 32 rows x
    // 4 kv heads x 576 keys with a cold L2: 65 us with 3 splits + merge, 74 us as one split
    const int64_t rows = kc.size(2);
    int splits = (int)std::min<int64_t>(std::max<int64_t>(1, (2 * 148 + B * G - 1) / (B * G)), std::max<int64_t>(1, rows / 128));
    splits = std::min(splits, 32);
    Tensor pa, pm;
    if (splits > 1) {
      pa = at::empty({B, H, splits, d}, qkvg.options().dtype(at::kFloat));
      pm = at::empty({B, H, splits, 2}, qkvg.options().dtype(at::kFloat));
    }
    const int rcf = rb_sink_window_decode_fast(qkvg.data_ptr(), qkvg.stride(0), out.data_ptr(), same_type_ptr(temp, qkvg, H, "temp"),
                                               same_type_ptr(sink, qkvg, H, "sink"), kc.data_ptr(), vc.data_ptr(), lens.data_ptr<int>(),
                                               int_ptr(slots, B, "slots"), splits > 1 ? pa.data_ptr<float>() : nullptr,
                                               splits > 1 ? pm.data_ptr<float>() : nullptr, splits, (int)B, (int)H, (int)G, (int)d, (int)rows, (float)scale,
                                               (int)window, (int)keep, (float)slope_base, gate ? 1 : 0, do_norm ? 1 : 0, (float)eps, dt_code(qkvg),
                                               (int)vshare, cur_stream());
    if (rcf == 0) return;
  }
  const int rc = rb_sink_window_decode(qkvg.data_ptr(), qkvg.stride(0), out.data_ptr(), same_type_ptr(temp, qkvg, H, "temp"),
                                       same_type_ptr(sink, qkvg, H, "sink"), kc.data_ptr(), vc.data_ptr(), lens.data_ptr<int>(), int_ptr(slots, B, "slots"),
                                       (int)B, (int)H, (int)G, (int)d, (int)dv, (int)kc.size(2), (float)scale, (int)window, (int)keep, (float)slope_base,
                                       gate ? 1 : 0, do_norm ? 1 : 0, (float)eps, dt_code(qkvg), (int)vshare, dt_code(out), cur_stream());
  TORCH_CHECK(rc == 0, "sink_window_decode_attention: unsupported shape (rc ", rc, ")");
}

// pos given: packed form (conv_state / tok_slot / remain optional); pos absent: step form (conv_state indexed by slots or row)
void delta_prepare(const Tensor& proj, const Tensor& conv_w, const Tensor& A_log, const Tensor& dt_bias, Tensor u, const OptT& pos, const OptT& conv_state,
                   const OptT& tok_slot, const OptT& remain, const OptT& slots, int64_t H, int64_t G, int64_t d, int64_t dv, int64_t taps,
                   double unit_eps) {
  CHECK_ROWS(proj); CHECK_IN(conv_w); CHECK_IN(A_log); CHECK_IN(dt_bias); CHECK_IN(u);
  const int64_t T = proj.size(0), C = 2 * G * d + H * dv;
  TORCH_CHECK(proj.size(1) >= C + H * dv + 2 * H && conv_w.numel() == C * taps && A_log.numel() == H && dt_bias.numel() == H);
  TORCH_CHECK(conv_w.scalar_type() == proj.scalar_type() && A_log.scalar_type() == proj.scalar_type() && dt_bias.scalar_type() == proj.scalar_type());
  TORCH_CHECK(u.scalar_type() == at::kFloat && u.numel() == T * (C + 2 * H));
  float* st = nullptr;
  if (conv_state.has_value() && taps > 1) {
    CHECK_IN((*conv_state));
    TORCH_CHECK(conv_state->scalar_type() == at::kFloat && conv_state->dim() == 3 && conv_state->size(1) == taps - 1 && conv_state->size(2) == C);
    TORCH_CHECK(pos.has_value() ? (tok_slot.has_value() && remain.has_value()) : (slots.has_value() || conv_state->size(0) >= T));
    st = conv_state->data_ptr<float>();
  }
  TORCH_CHECK(pos.has_value() || taps == 1 || st != nullptr, "the step form of a convolution needs its state");
  c10::cuda::CUDAGuard g(proj.device());
  const int rc = rb_delta_prepare(proj.data_ptr(), proj.stride(0), dt_code(proj), conv_w.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(),
                                  u.data_ptr<float>(), int_ptr(pos, T, "pos"), st, st && pos.has_value() ? int_ptr(tok_slot, T, "tok_slot") : nullptr,
                                  st && pos.has_value() ? int_ptr(remain, T, "remain") : nullptr, pos.has_value() ? nullptr : int_ptr(slots, T, "slots"),
                                  T, (int)H, (int)G, (int)d, (int)dv, (int)taps, (float)unit_eps, cur_stream());
  TORCH_CHECK(rc == 0, "delta_prepare: unsupported shape (rc ", rc, ")");
}

static void delta_rule(const Tensor& u, Tensor o, const int* cu, int n_seqs, const OptT& s_state, const OptT& slots, int64_t H, int64_t G, int64_t d,
                       int64_t dv, int step) {
  CHECK_IN(u); CHECK_IN(o);
  TORCH_CHECK(u.scalar_type() == at::kFloat && o.scalar_type() == at::kFloat && u.dim() == 2 && u.size(1) == 2 * G * d + H * dv + 2 * H);
  TORCH_CHECK(o.numel() == u.size(0) * H * dv);
  float* sp = nullptr;
  if (s_state.has_value()) {
    CHECK_IN((*s_state));
    TORCH_CHECK(s_state->scalar_type() == at::kFloat && s_state->dim() == 4 && s_state->size(1) == H && s_state->size(2) == d && s_state->size(3) == dv);
    TORCH_CHECK(slots.has_value() || (step && s_state->size(0) >= n_seqs));
    sp = s_state->data_ptr<float>();
  }
  TORCH_CHECK(!step || sp != nullptr, "the step form needs the state");
  c10::cuda::CUDAGuard g(u.device());
  const int rc = rb_delta_rule(u.data_ptr<float>(), o.data_ptr<float>(), cu, sp, int_ptr(slots, n_seqs, "slots"), n_seqs, (int)H, (int)G, (int)d, (int)dv,
                               step, cur_stream());
  TORCH_CHECK(rc == 0, "delta_rule: unsupported shape (rc ", rc, ")");
}

void delta_rule_scan(const Tensor& u, Tensor o, const Tensor& cu, const OptT& s_state, const OptT& slots, int64_t H, int64_t G, int64_t d, int64_t dv) {
  CHECK_IN(cu);
  TORCH_CHECK(cu.scalar_type() == at::kInt && cu.numel() >= 1);
  delta_rule(u, o, cu.data_ptr<int>(), (int)cu.numel() - 1, s_state, slots, H, G, d, dv, 0);
}

void delta_rule_step(const Tensor& u, Tensor o, Tensor s_state, const OptT& slots, int64_t H, int64_t G, int64_t d, int64_t dv) {
  delta_rule(u, o, nullptr, (int)u.size(0), s_state, slots, H, G, d, dv, 1);
}

void gated_head_norm(const Tensor& o, const Tensor& w, const Tensor& gate, Tensor out, double eps) {
  CHECK_IN(o); CHECK_IN(w); CHECK_ROWS(gate); CHECK_IN(out);
  TORCH_CHECK(o.dim() == 3 && o.scalar_type() == at::kFloat && w.numel() == o.size(2) && gate.size(0) == o.size(0) && gate.size(1) == o.size(1) * o.size(2));
  TORCH_CHECK(out.numel() == o.numel());
  c10::cuda::CUDAGuard g(o.device());
  TORCH_CHECK(rb_gated_head_norm(o.data_ptr<float>(), w.data_ptr(), dt_code(w), gate.data_ptr(), gate.stride(0), dt_code(gate), out.data_ptr(),
                                 dt_code(out), o.size(0), (int)o.size(1), (int)o.size(2), (float)eps, cur_stream()) == 0);
}

}  // namespace

void register_state_ops(torch::Library& m) {
  m.def("embed_sinusoid(Tensor ids, Tensor wte, Tensor pos, Tensor? slots, Tensor inv_freq, Tensor(a!) out) -> ()", &embed_sinusoid);
  m.def("concat_cast(Tensor a, Tensor b, Tensor(a!) out) -> ()", &concat_cast);
  m.def("relu2(Tensor x) -> Tensor", &relu2);
  m.def("rms_norm_rows(Tensor(a!) x, Tensor? y, Tensor w, Tensor(b!) out, float eps, float w_offset=0.0) -> ()", &rms_norm_rows);
  m.def("value_norm_store(Tensor qkvg, Tensor(a!) vout, Tensor(b!)? kc, Tensor(c!)? vc, Tensor? tok_slot, Tensor pos, Tensor? remain, int H, int G, int d, int dv, int keep, bool do_norm, float eps, int vshare=1) -> ()", &value_norm_store);
  m.def("sink_window_attention(Tensor qkvg, Tensor vn, Tensor(a!) out, Tensor? temp, Tensor? sink, Tensor cu, int max_seqlen, int H, int G, int d, int dv, float scale, int window, int keep, float slope_base, bool gate, int vshare=1) -> ()", &sink_window_attention);
  m.def("sink_window_attention_tc(Tensor qkvg, Tensor vn, Tensor(a!) out, Tensor? temp, Tensor? sink, Tensor cu, int max_seqlen, int H, int G, int d, float scale, int window, int keep, float slope_base, bool gate, int vshare=1) -> ()", &sink_window_attention_tc);
  m.def("sink_window_decode_attention(Tensor qkvg, Tensor(a!) out, Tensor? temp, Tensor? sink, Tensor(b!) kc, Tensor(c!) vc, Tensor lens, Tensor? slots, int H, int G, int d, int dv, float scale, int window, int keep, float slope_base, bool gate, bool do_norm, float eps, int vshare=1) -> ()", &sink_window_decode_attention);
  m.def("delta_prepare(Tensor proj, Tensor conv_w, Tensor A_log, Tensor dt_bias, Tensor(a!) u, Tensor? pos, Tensor(b!)? conv_state, Tensor? tok_slot, Tensor? remain, Tensor? slots, int H, int G, int d, int dv, int taps, float unit_eps) -> ()", &delta_prepare);
  m.def("delta_rule_scan(Tensor u, Tensor(a!) o, Tensor cu, Tensor(b!)? s_state, Tensor? slots, int H, int G, int d, int dv) -> ()", &delta_rule_scan);
  m.def("delta_rule_step(Tensor u, Tensor(a!) o, Tensor(b!) s_state, Tensor? slots, int H, int G, int d, int dv) -> ()", &delta_rule_step);
  m.def("gated_head_norm(Tensor o, Tensor w, Tensor gate, Tensor(a!) out, float eps) -> ()", &gated_head_norm);
}
