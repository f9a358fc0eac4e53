// Implementation of the C ABI declared in csrc/include/torsh.h: fp32 host tensors with the operation set of the
// reference's FFI layer (crates/torsh-ffi/src/c_api/*.rs), a linear layer with backward, SGD and Adam(W) with the
// reference arithmetic (crates/torsh-optim/src/sgd.rs:443-610, adam.rs:809-950). This is the portable surface other
// language bindings link against; GPU work goes through the Python package.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <map>
#include <string>
#include <cmath>
#include <cstring>
#include <functional>
#include <random>
#include <vector>

#include "host_api.h"
#include "torsh.h"

// Tensor storage is counted: torsh_get_memory_usage / torsh_get_peak_memory_usage report the bytes held by live
// tensors of this library (the reference keeps the same two counters, crates/torsh-ffi/src/c_api/utils.rs).
static std::atomic<size_t> g_mem_now{0}, g_mem_peak{0};
template <typename T>
struct CountingAlloc {
  using value_type = T;
  CountingAlloc() = default;
  template <typename U>
  CountingAlloc(const CountingAlloc<U>&) {}
  T* allocate(size_t n) {
    const size_t now = g_mem_now.fetch_add(n * sizeof(T)) + n * sizeof(T);
    size_t peak = g_mem_peak.load();
    while (now > peak && !g_mem_peak.compare_exchange_weak(peak, now)) {
    }
    return static_cast<T*>(::operator new(n * sizeof(T)));
  }
  void deallocate(T* p, size_t n) {
    g_mem_now.fetch_sub(n * sizeof(T));
    ::operator delete(p);
  }
  template <typename U>
  bool operator==(const CountingAlloc<U>&) const { return true; }
  template <typename U>
  bool operator!=(const CountingAlloc<U>&) const { return false; }
};

struct TorshTensor {
  std::vector<int64_t> shape;
  std::vector<float, CountingAlloc<float>> data;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};
struct TorshLinear {
  int64_t in, out;
  TorshTensor w, b, gw, gb, last_x;  // w: [in, out] as in the reference's Linear
  bool has_bias;
};
struct OptSlot {
  TorshTensor* p;
  TorshTensor* g;
  std::vector<float> m, v;
};
struct TorshOptimizer {
  int kind;  // 0 SGD, 1 Adam
  float lr, momentum, wd, b1, b2, eps;
  int nesterov, decoupled;
  int64_t t = 0;
  std::vector<OptSlot> slots;
};

namespace {
std::mt19937_64 g_rng(42);
bool g_grad = true;
#define EXPORT extern "C" __attribute__((visibility("default")))
TorshTensor* fail(const char* msg) {
  g_err = msg;
  return nullptr;
}
TorshTensor* make(const int64_t* shape, int ndim, float fill) {
  if (ndim < 0 || (ndim > 0 && !shape)) return fail("invalid shape");
  auto* t = new TorshTensor();
  t->shape.assign(shape, shape + ndim);
  for (auto d : t->shape)
    if (d < 0) { delete t; return fail("negative dimension"); }
  t->data.assign((size_t)t->numel(), fill);
  return t;
}
TorshTensor* unary(const TorshTensor* a, const std::function<float(float)>& f) {
  if (!a) return fail("null tensor");
  auto* o = new TorshTensor(*a);
  for (auto& x : o->data) x = f(x);
  return o;
}
TorshTensor* binary(const TorshTensor* a, const TorshTensor* b, const std::function<float(float, float)>& f) {
  if (!a || !b) return fail("null tensor");
  if (a->shape == b->shape) {
    auto* o = new TorshTensor(*a);
    for (size_t i = 0; i < o->data.size(); ++i) o->data[i] = f(a->data[i], b->data[i]);
    return o;
  }
  // broadcast of a trailing-dimension vector or a scalar
  if (b->numel() == 1) return unary(a, [&](float x) { return f(x, b->data[0]); });
  if (!a->shape.empty() && b->shape.size() == 1 && b->shape[0] == a->shape.back()) {
    auto* o = new TorshTensor(*a);
    int64_t n = b->shape[0];
    for (size_t i = 0; i < o->data.size(); ++i) o->data[i] = f(a->data[i], b->data[i % n]);
    return o;
  }
  return fail("shape mismatch: operands are neither equal-shaped nor broadcastable");
}
TorshTensor* reduce_all(const TorshTensor* a, int kind) {
  if (!a || a->data.empty()) return fail("null or empty tensor");
  double acc = kind == 2 ? -INFINITY : kind == 3 ? INFINITY : 0.0;
  for (float x : a->data) acc = kind == 2 ? std::max<double>(acc, x) : kind == 3 ? std::min<double>(acc, x) : acc + x;
  if (kind == 1) acc /= (double)a->data.size();
  auto* o = new TorshTensor();
  o->data = {(float)acc};
  return o;
}
}  // namespace

EXPORT TorshStatus torsh_init(void) { return 0; }
EXPORT void torsh_cleanup(void) {}
EXPORT const char* torsh_version(void) { return "0.1.0"; }
EXPORT const char* torsh_get_last_error(void) { return g_err.c_str(); }
EXPORT void torsh_set_random_seed(uint64_t seed) { g_rng.seed(seed); }
EXPORT void torsh_set_grad_enabled(int e) { g_grad = e != 0; }
EXPORT int torsh_is_grad_enabled(void) { return g_grad ? 1 : 0; }
EXPORT int torsh_cuda_is_available(void) { return 0; }  // the C surface computes on the host
EXPORT int torsh_cuda_device_count(void) { return 0; }
EXPORT TorshStatus torsh_set_device(int index) {
  if (index == 0) return 0;
  g_err = "only the host device is reachable through the C API";
  return 4;
}

EXPORT TorshTensor* torsh_tensor_new(const float* data, const int64_t* shape, int ndim) {
  TorshTensor* t = make(shape, ndim, 0.f);
  if (t && data) std::memcpy(t->data.data(), data, t->data.size() * sizeof(float));
  return t;
}
EXPORT TorshTensor* torsh_tensor_from_data(const float* d, const int64_t* s, int n) { return torsh_tensor_new(d, s, n); }
EXPORT TorshTensor* torsh_tensor_zeros(const int64_t* s, int n) { return make(s, n, 0.f); }
EXPORT TorshTensor* torsh_tensor_ones(const int64_t* s, int n) { return make(s, n, 1.f); }
EXPORT TorshTensor* torsh_tensor_rand(const int64_t* s, int n) {
  TorshTensor* t = make(s, n, 0.f);
  if (t) { std::uniform_real_distribution<float> d(0.f, 1.f); for (auto& x : t->data) x = d(g_rng); }
  return t;
}
EXPORT TorshTensor* torsh_tensor_randn(const int64_t* s, int n) {
  TorshTensor* t = make(s, n, 0.f);
  if (t) { std::normal_distribution<float> d(0.f, 1.f); for (auto& x : t->data) x = d(g_rng); }
  return t;
}
EXPORT TorshTensor* torsh_tensor_clone(const TorshTensor* t) { return t ? new TorshTensor(*t) : fail("null tensor"); }
EXPORT TorshTensor* torsh_tensor_detach(const TorshTensor* t) { return torsh_tensor_clone(t); }
EXPORT void torsh_tensor_free(TorshTensor* t) { delete t; }
EXPORT float* torsh_tensor_data(TorshTensor* t) { return t ? t->data.data() : nullptr; }
EXPORT int torsh_tensor_ndim(const TorshTensor* t) { return t ? (int)t->shape.size() : -1; }
EXPORT int64_t torsh_tensor_numel(const TorshTensor* t) { return t ? t->numel() : -1; }
EXPORT int torsh_tensor_dtype(const TorshTensor*) { return 0; }
EXPORT TorshStatus torsh_tensor_shape(const TorshTensor* t, int64_t* out, int cap) {
  if (!t || !out || cap < (int)t->shape.size()) { g_err = "shape buffer too small"; return 1; }
  std::copy(t->shape.begin(), t->shape.end(), out);
  return 0;
}

EXPORT TorshTensor* torsh_tensor_add(const TorshTensor* a, const TorshTensor* b) { return binary(a, b, [](float x, float y) { return x + y; }); }
EXPORT TorshTensor* torsh_tensor_sub(const TorshTensor* a, const TorshTensor* b) { return binary(a, b, [](float x, float y) { return x - y; }); }
EXPORT TorshTensor* torsh_tensor_mul(const TorshTensor* a, const TorshTensor* b) { return binary(a, b, [](float x, float y) { return x * y; }); }
EXPORT TorshTensor* torsh_tensor_div(const TorshTensor* a, const TorshTensor* b) { return binary(a, b, [](float x, float y) { return x / y; }); }
EXPORT TorshTensor* torsh_tensor_add_scalar(const TorshTensor* a, float s) { return unary(a, [s](float x) { return x + s; }); }
EXPORT TorshTensor* torsh_tensor_mul_scalar(const TorshTensor* a, float s) { return unary(a, [s](float x) { return x * s; }); }
EXPORT TorshTensor* torsh_tensor_relu(const TorshTensor* a) { return unary(a, [](float x) { return x > 0 ? x : 0.f; }); }
EXPORT TorshTensor* torsh_tensor_sigmoid(const TorshTensor* a) { return unary(a, [](float x) { return 1.f / (1.f + std::exp(-x)); }); }
EXPORT TorshTensor* torsh_tensor_tanh(const TorshTensor* a) { return unary(a, [](float x) { return std::tanh(x); }); }
EXPORT TorshTensor* torsh_tensor_exp(const TorshTensor* a) { return unary(a, [](float x) { return std::exp(x); }); }
EXPORT TorshTensor* torsh_tensor_log(const TorshTensor* a) { return unary(a, [](float x) { return std::log(x); }); }
EXPORT TorshTensor* torsh_tensor_sqrt(const TorshTensor* a) { return unary(a, [](float x) { return std::sqrt(x); }); }
EXPORT TorshTensor* torsh_tensor_abs(const TorshTensor* a) { return unary(a, [](float x) { return std::fabs(x); }); }
EXPORT TorshTensor* torsh_tensor_sin(const TorshTensor* a) { return unary(a, [](float x) { return std::sin(x); }); }
EXPORT TorshTensor* torsh_tensor_cos(const TorshTensor* a) { return unary(a, [](float x) { return std::cos(x); }); }
EXPORT TorshTensor* torsh_tensor_sum_all(const TorshTensor* a) { return reduce_all(a, 0); }
EXPORT TorshTensor* torsh_tensor_mean_all(const TorshTensor* a) { return reduce_all(a, 1); }
EXPORT TorshTensor* torsh_tensor_max_all(const TorshTensor* a) { return reduce_all(a, 2); }
EXPORT TorshTensor* torsh_tensor_min_all(const TorshTensor* a) { return reduce_all(a, 3); }

EXPORT TorshTensor* torsh_tensor_matmul(const TorshTensor* a, const TorshTensor* b) {
  if (!a || !b || a->shape.size() != 2 || b->shape.size() != 2) return fail("matmul expects two 2-D tensors");
  int64_t M = a->shape[0], K = a->shape[1], N = b->shape[1];
  if (b->shape[0] != K) return fail("shape mismatch: inner dimensions differ");
  auto* o = new TorshTensor();
  o->shape = {M, N};
  o->data.assign((size_t)(M * N), 0.f);
  for (int64_t i = 0; i < M; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const float x = a->data[i * K + k];
      const float* br = &b->data[k * N];
      float* orow = &o->data[i * N];
      for (int64_t j = 0; j < N; ++j) orow[j] += x * br[j];
    }
  return o;
}
EXPORT TorshTensor* torsh_tensor_reshape(const TorshTensor* a, const int64_t* shape, int ndim) {
  if (!a) return fail("null tensor");
  int64_t n = 1;
  for (int i = 0; i < ndim; ++i) n *= shape[i];
  if (n != a->numel()) return fail("shape mismatch: reshape changes the number of elements");
  auto* o = new TorshTensor(*a);
  o->shape.assign(shape, shape + ndim);
  return o;
}
EXPORT TorshTensor* torsh_tensor_transpose(const TorshTensor* a, int d0, int d1) {
  if (!a) return fail("null tensor");
  int nd = (int)a->shape.size();
  if (d0 < 0) d0 += nd;
  if (d1 < 0) d1 += nd;
  if (d0 < 0 || d1 < 0 || d0 >= nd || d1 >= nd) return fail("transpose dimension out of range");
  auto* o = new TorshTensor();
  o->shape = a->shape;
  std::swap(o->shape[d0], o->shape[d1]);
  o->data.resize(a->data.size());
  std::vector<int64_t> st(nd, 1), ost(nd, 1);
  for (int i = nd - 2; i >= 0; --i) { st[i] = st[i + 1] * a->shape[i + 1]; ost[i] = ost[i + 1] * o->shape[i + 1]; }
  std::vector<int64_t> idx(nd);
  for (int64_t lin = 0; lin < (int64_t)a->data.size(); ++lin) {
    int64_t r = lin;
    for (int i = 0; i < nd; ++i) { idx[i] = r / st[i]; r %= st[i]; }
    std::swap(idx[d0], idx[d1]);
    int64_t dst = 0;
    for (int i = 0; i < nd; ++i) dst += idx[i] * ost[i];
    o->data[dst] = a->data[lin];
  }
  return o;
}
static TorshTensor* reduce_dim(const TorshTensor* a, int dim, int keepdim, bool mean) {
  if (!a) return fail("null tensor");
  int nd = (int)a->shape.size();
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) return fail("reduction dimension out of range");
  int64_t outer = 1, axis = a->shape[dim], inner = 1;
  for (int i = 0; i < dim; ++i) outer *= a->shape[i];
  for (int i = dim + 1; i < nd; ++i) inner *= a->shape[i];
  auto* o = new TorshTensor();
  for (int i = 0; i < nd; ++i) {
    if (i == dim) { if (keepdim) o->shape.push_back(1); }
    else o->shape.push_back(a->shape[i]);
  }
  o->data.assign((size_t)(outer * inner), 0.f);
  for (int64_t x = 0; x < outer; ++x)
    for (int64_t k = 0; k < axis; ++k)
      for (int64_t y = 0; y < inner; ++y) o->data[x * inner + y] += a->data[(x * axis + k) * inner + y];
  if (mean) for (auto& v : o->data) v /= (float)axis;
  return o;
}
EXPORT TorshTensor* torsh_tensor_sum_dim(const TorshTensor* a, int dim, int keepdim) { return reduce_dim(a, dim, keepdim, false); }
EXPORT TorshTensor* torsh_tensor_mean_dim(const TorshTensor* a, int dim, int keepdim) { return reduce_dim(a, dim, keepdim, true); }
EXPORT TorshTensor* torsh_tensor_softmax(const TorshTensor* a, int dim) {
  if (!a) return fail("null tensor");
  int nd = (int)a->shape.size();
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) return fail("softmax dimension out of range");
  int64_t outer = 1, axis = a->shape[dim], inner = 1;
  for (int i = 0; i < dim; ++i) outer *= a->shape[i];
  for (int i = dim + 1; i < nd; ++i) inner *= a->shape[i];
  auto* o = new TorshTensor(*a);
  for (int64_t x = 0; x < outer; ++x)
    for (int64_t y = 0; y < inner; ++y) {
      float m = -INFINITY, s = 0.f;
      for (int64_t k = 0; k < axis; ++k) m = std::max(m, a->data[(x * axis + k) * inner + y]);
      for (int64_t k = 0; k < axis; ++k) { float e = std::exp(a->data[(x * axis + k) * inner + y] - m); o->data[(x * axis + k) * inner + y] = e; s += e; }
      for (int64_t k = 0; k < axis; ++k) o->data[(x * axis + k) * inner + y] /= s;
    }
  return o;
}
EXPORT TorshTensor* torsh_tensor_conv2d(const TorshTensor* in, const TorshTensor* w, const TorshTensor* bias, int stride, int pad) {
  if (!in || !w || in->shape.size() != 4 || w->shape.size() != 4) return fail("conv2d expects [N,C,H,W] and [O,C,kh,kw]");
  int64_t N = in->shape[0], C = in->shape[1], H = in->shape[2], W = in->shape[3], O = w->shape[0], kh = w->shape[2], kw = w->shape[3];
  if (w->shape[1] != C || stride < 1) return fail("shape mismatch: conv2d channels / stride");
  int64_t Ho = (H + 2 * pad - kh) / stride + 1, Wo = (W + 2 * pad - kw) / stride + 1;
  auto* o = new TorshTensor();
  o->shape = {N, O, Ho, Wo};
  o->data.assign((size_t)(N * O * Ho * Wo), 0.f);
  for (int64_t n = 0; n < N; ++n) for (int64_t oc = 0; oc < O; ++oc) for (int64_t y = 0; y < Ho; ++y) for (int64_t x = 0; x < Wo; ++x) {
    float acc = bias ? bias->data[oc] : 0.f;
    for (int64_t c = 0; c < C; ++c) for (int64_t i = 0; i < kh; ++i) for (int64_t j = 0; j < kw; ++j) {
      int64_t yy = y * stride - pad + i, xx = x * stride - pad + j;
      if (yy >= 0 && yy < H && xx >= 0 && xx < W) acc += in->data[((n * C + c) * H + yy) * W + xx] * w->data[((oc * C + c) * kh + i) * kw + j];
    }
    o->data[((n * O + oc) * Ho + y) * Wo + x] = acc;
  }
  return o;
}

// ---- linear layer: weight [in, out], y = x W + b, Xavier-uniform init, zero bias --------------------------
EXPORT TorshLinear* torsh_linear_new(int64_t in, int64_t out, int bias) {
  if (in <= 0 || out <= 0) { g_err = "linear: sizes must be positive"; return nullptr; }
  auto* l = new TorshLinear();
  l->in = in; l->out = out; l->has_bias = bias != 0;
  l->w.shape = {in, out}; l->w.data.resize((size_t)(in * out));
  float a = std::sqrt(6.f / (float)(in + out));
  std::uniform_real_distribution<float> d(-a, a);
  for (auto& x : l->w.data) x = d(g_rng);
  l->gw.shape = l->w.shape; l->gw.data.assign(l->w.data.size(), 0.f);
  l->b.shape = {out}; l->b.data.assign((size_t)out, 0.f);
  l->gb.shape = {out}; l->gb.data.assign((size_t)out, 0.f);
  return l;
}
EXPORT TorshTensor* torsh_linear_forward(TorshLinear* l, const TorshTensor* x) {
  if (!l || !x || x->shape.empty() || x->shape.back() != l->in) return fail("linear: input feature size mismatch");
  TorshTensor x2 = *x;
  x2.shape = {x->numel() / l->in, l->in};
  if (g_grad) l->last_x = x2;
  TorshTensor* y = torsh_tensor_matmul(&x2, &l->w);
  if (l->has_bias) for (size_t i = 0; i < y->data.size(); ++i) y->data[i] += l->b.data[i % l->out];
  y->shape = x->shape;
  y->shape.back() = l->out;
  return y;
}
EXPORT TorshTensor* torsh_linear_backward(TorshLinear* l, const TorshTensor* gy) {
  if (!l || !gy || l->last_x.data.empty()) return fail("linear: backward without a recorded forward");
  int64_t M = l->last_x.shape[0];
  if (gy->numel() != M * l->out) return fail("shape mismatch: grad_output");
  for (int64_t i = 0; i < M; ++i)
    for (int64_t k = 0; k < l->in; ++k) {
      float x = l->last_x.data[i * l->in + k];
      for (int64_t j = 0; j < l->out; ++j) l->gw.data[k * l->out + j] += x * gy->data[i * l->out + j];
    }
  if (l->has_bias) for (int64_t i = 0; i < M; ++i) for (int64_t j = 0; j < l->out; ++j) l->gb.data[j] += gy->data[i * l->out + j];
  auto* gx = new TorshTensor();
  gx->shape = l->last_x.shape;
  gx->data.assign((size_t)(M * l->in), 0.f);
  for (int64_t i = 0; i < M; ++i) for (int64_t k = 0; k < l->in; ++k) {
    float acc = 0.f;
    for (int64_t j = 0; j < l->out; ++j) acc += gy->data[i * l->out + j] * l->w.data[k * l->out + j];
    gx->data[i * l->in + k] = acc;
  }
  return gx;
}
EXPORT TorshTensor* torsh_linear_weight(TorshLinear* l) { return l ? &l->w : nullptr; }
EXPORT TorshTensor* torsh_linear_bias(TorshLinear* l) { return l && l->has_bias ? &l->b : nullptr; }
EXPORT void torsh_linear_free(TorshLinear* l) { delete l; }

// ---- optimizers -------------------------------------------------------------------------------------------
EXPORT TorshOptimizer* torsh_sgd_new(float lr, float momentum, float wd, int nesterov) {
  auto* o = new TorshOptimizer();
  o->kind = 0; o->lr = lr; o->momentum = momentum; o->wd = wd; o->nesterov = nesterov; o->b1 = o->b2 = o->eps = 0; o->decoupled = 0;
  return o;
}
EXPORT TorshOptimizer* torsh_adam_new(float lr, float b1, float b2, float eps, float wd, int decoupled) {
  auto* o = new TorshOptimizer();
  o->kind = 1; o->lr = lr; o->b1 = b1; o->b2 = b2; o->eps = eps; o->wd = wd; o->decoupled = decoupled; o->momentum = 0; o->nesterov = 0;
  return o;
}
EXPORT TorshStatus torsh_optimizer_add_linear(TorshOptimizer* o, TorshLinear* l) {
  if (!o || !l) { g_err = "null handle"; return 1; }
  o->slots.push_back({&l->w, &l->gw, std::vector<float>(l->w.data.size(), 0.f), std::vector<float>(l->w.data.size(), 0.f)});
  if (l->has_bias) o->slots.push_back({&l->b, &l->gb, std::vector<float>(l->b.data.size(), 0.f), std::vector<float>(l->b.data.size(), 0.f)});
  return 0;
}
EXPORT TorshStatus torsh_optimizer_step(TorshOptimizer* o) {
  if (!o) { g_err = "null handle"; return 1; }
  o->t += 1;
  for (auto& s : o->slots)
    for (size_t i = 0; i < s.p->data.size(); ++i) {
      float p = s.p->data[i], g = s.g->data[i];
      if (o->kind == 0) {
        float d = g + o->wd * p;
        if (o->momentum != 0.f) { s.m[i] = o->momentum * s.m[i] + d; d = o->nesterov ? d + o->momentum * s.m[i] : s.m[i]; }
        p -= o->lr * d;
      } else {
        if (o->decoupled) p -= o->lr * o->wd * p; else g += o->wd * p;
        s.m[i] = o->b1 * s.m[i] + (1 - o->b1) * g;
        s.v[i] = o->b2 * s.v[i] + (1 - o->b2) * g * g;
        float mh = s.m[i] / (1 - std::pow(o->b1, (float)o->t)), vh = s.v[i] / (1 - std::pow(o->b2, (float)o->t));
        p -= o->lr * mh / (std::sqrt(vh) + o->eps);
      }
      s.p->data[i] = p;
    }
  return 0;
}
EXPORT TorshStatus torsh_optimizer_zero_grad(TorshOptimizer* o) {
  if (!o) { g_err = "null handle"; return 1; }
  for (auto& s : o->slots) std::fill(s.g->data.begin(), s.g->data.end(), 0.f);
  return 0;
}
EXPORT void torsh_optimizer_free(TorshOptimizer* o) { delete o; }

// ---- the rest of the reference's C surface (crates/torsh-ffi/src/c_api/{tensor,tensor_math,neural,optimizer,utils}.rs) -----
namespace {
int g_threads = 1;
bool g_autocast = false, g_debug = false, g_profiling = false;
std::chrono::steady_clock::time_point g_prof_start;
std::string g_prof_json;
struct StandaloneState {            // optimizers created without layers step explicit tensors (torsh_*_step_inplace)
  float lr, b1, b2, eps;
};
}  // namespace

EXPORT void torsh_clear_last_error(void) { g_err.clear(); }
EXPORT int torsh_has_error(void) { return g_err.empty() ? 0 : 1; }
EXPORT int torsh_get_device_type(void) { return 0; }  // 0 = host: the C surface computes on the host
EXPORT int torsh_get_device_id(void) { return 0; }
EXPORT size_t torsh_cuda_device_memory(int) { return 0; }
EXPORT const char* torsh_cuda_device_name(int) { return ""; }
EXPORT size_t torsh_get_memory_usage(void) { return g_mem_now.load(); }
EXPORT size_t torsh_get_peak_memory_usage(void) { return g_mem_peak.load(); }
EXPORT TorshStatus torsh_reset_memory_tracking(void) {
  g_mem_peak.store(g_mem_now.load());
  return 0;
}
EXPORT int torsh_get_num_threads(void) { return g_threads; }
EXPORT TorshStatus torsh_set_num_threads(int n) {
  if (n < 1) { g_err = "thread count must be positive"; return 1; }
  g_threads = n;
  return 0;
}
EXPORT TorshStatus torsh_set_autocast(int e) { g_autocast = e != 0; return 0; }
EXPORT int torsh_is_autocast_enabled(void) { return g_autocast ? 1 : 0; }
EXPORT TorshStatus torsh_set_debug_mode(int e) { g_debug = e != 0; return 0; }
EXPORT int torsh_is_debug_mode_enabled(void) { return g_debug ? 1 : 0; }
EXPORT TorshStatus torsh_start_profiling(void) {
  g_profiling = true;
  g_prof_start = std::chrono::steady_clock::now();
  return 0;
}
// JSON object {"elapsed_ms": ..., "memory_bytes": ..., "peak_memory_bytes": ...}; the string stays valid until the next call.
EXPORT const char* torsh_stop_profiling(void) {
  if (!g_profiling) return "";
  g_profiling = false;
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - g_prof_start).count();
  g_prof_json = "{\"elapsed_ms\": " + std::to_string(ms) + ", \"memory_bytes\": " + std::to_string(g_mem_now.load()) +
                ", \"peak_memory_bytes\": " + std::to_string(g_mem_peak.load()) + "}";
  return g_prof_json.c_str();
}

EXPORT size_t torsh_tensor_size(const TorshTensor* t) { return t ? (size_t)t->numel() : 0; }
EXPORT TorshTensor* torsh_tensor_scalar(float v) {
  auto* t = new TorshTensor();
  t->data = {v};
  return t;
}
EXPORT TorshTensor* torsh_tensor_eye(size_t n) {
  int64_t shape[2] = {(int64_t)n, (int64_t)n};
  TorshTensor* t = make(shape, 2, 0.f);
  if (t) for (size_t i = 0; i < n; ++i) t->data[i * n + i] = 1.f;
  return t;
}
EXPORT TorshTensor* torsh_tensor_linspace(double start, double end, size_t steps) {
  if (steps == 0) return fail("linspace: steps must be positive");
  int64_t shape[1] = {(int64_t)steps};
  TorshTensor* t = make(shape, 1, 0.f);
  if (t) for (size_t i = 0; i < steps; ++i) t->data[i] = (float)(steps == 1 ? start : start + (end - start) * (double)i / (double)(steps - 1));
  return t;
}
EXPORT TorshTensor* torsh_tensor_sub_scalar(const TorshTensor* a, float s) { return unary(a, [s](float x) { return x - s; }); }
EXPORT TorshTensor* torsh_tensor_div_scalar(const TorshTensor* a, float s) {
  if (s == 0.f) return fail("division by zero");
  return unary(a, [s](float x) { return x / s; });
}
EXPORT TorshTensor* torsh_tensor_tan(const TorshTensor* a) { return unary(a, [](float x) { return std::tan(x); }); }
// result = a * b element-wise into an existing tensor of the same shape.
EXPORT TorshStatus torsh_tensor_multiply(const TorshTensor* a, const TorshTensor* b, TorshTensor* result) {
  if (!a || !b || !result) { g_err = "null tensor"; return 1; }
  if (a->shape != b->shape || a->shape != result->shape) { g_err = "shape mismatch"; return 2; }
  for (size_t i = 0; i < a->data.size(); ++i) result->data[i] = a->data[i] * b->data[i];
  return 0;
}
static TorshTensor* extreme_dim(const TorshTensor* a, int dim, bool want_max) {
  if (!a) return fail("null tensor");
  const int nd = (int)a->shape.size();
  if (nd == 0) return reduce_all(a, want_max ? 2 : 3);
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) return fail("dimension out of range");
  int64_t outer = 1, inner = 1;
  const int64_t n = a->shape[dim];
  if (n == 0) return fail("cannot reduce an empty dimension");
  for (int i = 0; i < dim; ++i) outer *= a->shape[i];
  for (int i = dim + 1; i < nd; ++i) inner *= a->shape[i];
  auto* o = new TorshTensor();
  o->shape = a->shape;
  o->shape.erase(o->shape.begin() + dim);
  o->data.assign((size_t)(outer * inner), 0.f);
  for (int64_t u = 0; u < outer; ++u)
    for (int64_t v = 0; v < inner; ++v) {
      float best = a->data[(u * n) * inner + v];
      for (int64_t k = 1; k < n; ++k) {
        const float x = a->data[(u * n + k) * inner + v];
        best = want_max ? std::max(best, x) : std::min(best, x);
      }
      o->data[u * inner + v] = best;
    }
  return o;
}
// The reference ignores `dim` here and returns the global extreme (tensor_math.rs); this reduces along `dim`.
EXPORT TorshTensor* torsh_tensor_max_dim(const TorshTensor* a, int dim) { return extreme_dim(a, dim, true); }
EXPORT TorshTensor* torsh_tensor_min_dim(const TorshTensor* a, int dim) { return extreme_dim(a, dim, false); }
// target += alpha * source
EXPORT TorshStatus torsh_tensor_axpy_inplace(TorshTensor* target, const TorshTensor* source, float alpha) {
  if (!target || !source) { g_err = "null tensor"; return 1; }
  if (target->data.size() != source->data.size()) { g_err = "shape mismatch"; return 2; }
  for (size_t i = 0; i < target->data.size(); ++i) target->data[i] += alpha * source->data[i];
  return 0;
}
// One Adam step on explicit tensors (no weight decay), bias-corrected with `step` (1-based).
EXPORT TorshStatus torsh_tensor_adam_step_inplace(TorshTensor* param, const TorshTensor* grad, TorshTensor* m, TorshTensor* v,
                                                  float lr, float beta1, float beta2, float eps, int64_t step) {
  if (!param || !grad || !m || !v) { g_err = "null tensor"; return 1; }
  const size_t n = param->data.size();
  if (grad->data.size() != n || m->data.size() != n || v->data.size() != n) { g_err = "shape mismatch"; return 2; }
  if (step < 1) { g_err = "step must be >= 1"; return 1; }
  const float c1 = 1.f - std::pow(beta1, (float)step), c2 = 1.f - std::pow(beta2, (float)step);
  for (size_t i = 0; i < n; ++i) {
    const float g = grad->data[i];
    m->data[i] = beta1 * m->data[i] + (1.f - beta1) * g;
    v->data[i] = beta2 * v->data[i] + (1.f - beta2) * g * g;
    param->data[i] -= lr * (m->data[i] / c1) / (std::sqrt(v->data[i] / c2) + eps);
  }
  return 0;
}

// Reference-named constructors / accessors: a "module" of the C surface is the linear layer.
EXPORT TorshModule* torsh_linear_create(size_t in_features, size_t out_features, bool bias) {
  return torsh_linear_new((int64_t)in_features, (int64_t)out_features, bias ? 1 : 0);
}
EXPORT size_t torsh_linear_get_input_features(const TorshModule* m) { return m ? (size_t)m->in : 0; }
EXPORT size_t torsh_linear_get_output_features(const TorshModule* m) { return m ? (size_t)m->out : 0; }
EXPORT void torsh_module_free(TorshModule* m) { delete m; }
EXPORT TorshOptimizer* torsh_sgd_create(float lr) { return torsh_sgd_new(lr, 0.f, 0.f, 0); }
EXPORT TorshOptimizer* torsh_adam_create(float lr, float beta1, float beta2, float eps) {
  return torsh_adam_new(lr, beta1, beta2, eps, 0.f, 0);
}
// Steps the parameters registered with torsh_optimizer_add_linear (the reference's version is a no-op that returns
// success, optimizer.rs); refuses an optimizer of the other kind.
EXPORT TorshStatus torsh_sgd_step(TorshOptimizer* o) {
  if (!o || o->kind != 0) { g_err = "not an SGD optimizer"; return 1; }
  return torsh_optimizer_step(o);
}
