// C++ host mirror of cleave's tensor operator surface over the C ABI of cleave_cuda.h (header only).
//
// The reference's surface is the cleave standard library:
//   struct Tensor<T: Float, const Dims...: i32>                    stdlib/linalg/tensor.cleave:40
//   Ring<Tensor>::{add, sub, mul, div, neg, zero}                  stdlib/linalg/tensor.cleave:66-80
//   MatMul<Tensor<T,N,M>, Tensor<T,M,K>, Tensor<T,N,K>>::matmul    stdlib/linalg/matrix.cleave:22-62
//   Activation::{relu, sigmoid, tanh}, Transcendental::exp         stdlib/nn/nn.cleave:54-95, stdlib/num/num.cleave:218-234
//   Sum / Mean / Max, Index                                        stdlib/nn/nn.cleave:111-149, stdlib/linalg/tensor.cleave:129-133
// The same names, the static shape in the type, shape errors at compile time.  Differences a caller sees:
// values live in device memory (construction uploads, `to_host` / `at` read back), handles are freed when the
// value dies (cleave's runtime never frees), and a failed call throws `cleave_cuda::Error` where the
// reference's runtime would abort.
#pragma once
#include <array>
#include <cstdint>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#include "cleave_cuda.h"

namespace cleave_cuda {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};

inline void throw_last(const char* what) {
  const int code = cleave_cuda_last_error();
  const char* msg = cleave_cuda_last_error_message();
  std::string text = std::string(what) + ": " + (msg ? msg : "");
  cleave_cuda_clear_error();
  throw Error(code, text);
}

namespace detail {
template <int... Dims>
constexpr int64_t numel() { return (int64_t(1) * ... * Dims); }

// per-dtype entry points, selected by overload on a tag value
inline cleave_buf upload(const float* p, int64_t n) { return cleave_cuda_upload_f32(p, n); }
inline cleave_buf upload(const double* p, int64_t n) { return cleave_cuda_upload_f64(p, n); }
inline int64_t download(cleave_buf h, float* p, int64_t n) { return cleave_cuda_download_f32(h, p, n); }
inline int64_t download(cleave_buf h, double* p, int64_t n) { return cleave_cuda_download_f64(h, p, n); }
inline cleave_buf zeros(float, int64_t n) { return cleave_cuda_zeros_f32(n); }
inline cleave_buf zeros(double, int64_t n) { return cleave_cuda_zeros_f64(n); }
inline cleave_buf fill(float v, int64_t n) { return cleave_cuda_fill_f32(v, n); }
inline cleave_buf fill(double v, int64_t n) { return cleave_cuda_fill_f64(v, n); }
inline float get(float, cleave_buf h, int64_t i) { return cleave_cuda_get_f32(h, i); }
inline double get(double, cleave_buf h, int64_t i) { return cleave_cuda_get_f64(h, i); }

#define CLEAVE_CUDA_BINARY(NAME)                                                                         \
  inline cleave_buf NAME(float, cleave_buf a, cleave_buf b) { return cleave_cuda_##NAME##_f32(a, b); }   \
  inline cleave_buf NAME(double, cleave_buf a, cleave_buf b) { return cleave_cuda_##NAME##_f64(a, b); }
CLEAVE_CUDA_BINARY(add)
CLEAVE_CUDA_BINARY(sub)
CLEAVE_CUDA_BINARY(mul)
CLEAVE_CUDA_BINARY(div)
#undef CLEAVE_CUDA_BINARY
#define CLEAVE_CUDA_UNARY(NAME)                                                            \
  inline cleave_buf NAME(float, cleave_buf a) { return cleave_cuda_##NAME##_f32(a); }      \
  inline cleave_buf NAME(double, cleave_buf a) { return cleave_cuda_##NAME##_f64(a); }
CLEAVE_CUDA_UNARY(neg)
CLEAVE_CUDA_UNARY(relu)
CLEAVE_CUDA_UNARY(sigmoid)
CLEAVE_CUDA_UNARY(tanh)
CLEAVE_CUDA_UNARY(exp)
#undef CLEAVE_CUDA_UNARY
#define CLEAVE_CUDA_REDUCE(NAME)                                                  \
  inline float NAME(float, cleave_buf a) { return cleave_cuda_##NAME##_f32(a); }  \
  inline double NAME(double, cleave_buf a) { return cleave_cuda_##NAME##_f64(a); }
CLEAVE_CUDA_REDUCE(sum)
CLEAVE_CUDA_REDUCE(mean)
CLEAVE_CUDA_REDUCE(max)
#undef CLEAVE_CUDA_REDUCE
inline cleave_buf gemm(float, cleave_buf a, cleave_buf b, int m, int n, int k) { return cleave_cuda_gemm_f32(a, b, m, n, k); }
inline cleave_buf gemm(double, cleave_buf a, cleave_buf b, int m, int n, int k) { return cleave_cuda_gemm_f64(a, b, m, n, k); }
}  // namespace detail

// Dense, row-major, static-shape device tensor; an immutable value like cleave's Tensor.
template <class T, int... Dims>
class Tensor {
  static_assert(std::is_same<T, float>::value || std::is_same<T, double>::value, "T: Float means f32 or f64");
  static_assert(sizeof...(Dims) >= 1 && ((Dims > 0) && ...), "every dimension must be positive");

 public:
  static constexpr int64_t size = detail::numel<Dims...>();

  // Tensor::<T, Dims...>(data: [...]): row-major values
  explicit Tensor(const std::vector<T>& data) : h_(nullptr) {
    if ((int64_t)data.size() != size) throw Error(CLEAVE_CUDA_ERR_SHAPE, "Tensor: data length does not match the shape");
    h_ = detail::upload(data.data(), size);
    if (!h_) throw_last("Tensor");
  }
  Tensor(std::initializer_list<T> data) : Tensor(std::vector<T>(data)) {}
  // Ring::zero and the filled form (tests/mlir_lower.rs:2161-2184 build tensors of one value)
  static Tensor zero() { return adopt(detail::zeros(T(), size), "zero"); }
  static Tensor filled(T v) { return adopt(detail::fill(v, size), "filled"); }

  Tensor(const Tensor&) = delete;   // a value is one device buffer; copy explicitly with clone()
  Tensor& operator=(const Tensor&) = delete;
  Tensor(Tensor&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
  Tensor& operator=(Tensor&& o) noexcept {
    if (this != &o) { release(); h_ = o.h_; o.h_ = nullptr; }
    return *this;
  }
  ~Tensor() { release(); }

  Tensor clone() const { return *this + zero(); }
  cleave_buf handle() const { return h_; }

  std::vector<T> to_host() const {
    std::vector<T> out(size);
    if (detail::download(h_, out.data(), size) < 0) throw_last("to_host");
    return out;
  }
  // Index::index(t, [i, j, ...]) (stdlib/linalg/tensor.cleave:129-133)
  template <class... I>
  T at(I... idx) const {
    static_assert(sizeof...(I) == sizeof...(Dims), "one index per dimension");
    const int64_t ix[] = {int64_t(idx)...};
    const int64_t dm[] = {int64_t(Dims)...};
    int64_t flat = 0;
    for (size_t d = 0; d < sizeof...(Dims); ++d) {
      if (ix[d] < 0 || ix[d] >= dm[d]) throw Error(CLEAVE_CUDA_ERR_ARG, "index out of range");
      flat = flat * dm[d] + ix[d];
    }
    const T v = detail::get(T(), h_, flat);
    if (v != v && cleave_cuda_last_error() != 0) throw_last("index");
    return v;
  }

  // Ring<Tensor>
  friend Tensor operator+(const Tensor& a, const Tensor& b) { return adopt(detail::add(T(), a.h_, b.h_), "add"); }
  friend Tensor operator-(const Tensor& a, const Tensor& b) { return adopt(detail::sub(T(), a.h_, b.h_), "sub"); }
  friend Tensor operator*(const Tensor& a, const Tensor& b) { return adopt(detail::mul(T(), a.h_, b.h_), "mul"); }
  friend Tensor operator/(const Tensor& a, const Tensor& b) { return adopt(detail::div(T(), a.h_, b.h_), "div"); }
  friend Tensor operator-(const Tensor& a) { return adopt(detail::neg(T(), a.h_), "neg"); }

  static Tensor adopt(cleave_buf h, const char* what) {
    if (!h) throw_last(what);
    Tensor t;
    t.h_ = h;
    return t;
  }

 private:
  Tensor() : h_(nullptr) {}
  void release() {
    if (h_) cleave_cuda_free(h_);
    h_ = nullptr;
  }
  cleave_buf h_;
};

// MatMul: Tensor<T,N,M> x Tensor<T,M,K> -> Tensor<T,N,K>; a shape mismatch does not compile.
template <class T, int N, int M, int K>
Tensor<T, N, K> matmul(const Tensor<T, N, M>& a, const Tensor<T, M, K>& b) {
  return Tensor<T, N, K>::adopt(detail::gemm(T(), a.handle(), b.handle(), N, K, M), "matmul");
}

// Activation / Transcendental, on tensors of any rank
template <class T, int... D> Tensor<T, D...> relu(const Tensor<T, D...>& x) { return Tensor<T, D...>::adopt(detail::relu(T(), x.handle()), "relu"); }
template <class T, int... D> Tensor<T, D...> sigmoid(const Tensor<T, D...>& x) { return Tensor<T, D...>::adopt(detail::sigmoid(T(), x.handle()), "sigmoid"); }
template <class T, int... D> Tensor<T, D...> tanh(const Tensor<T, D...>& x) { return Tensor<T, D...>::adopt(detail::tanh(T(), x.handle()), "tanh"); }
template <class T, int... D> Tensor<T, D...> exp(const Tensor<T, D...>& x) { return Tensor<T, D...>::adopt(detail::exp(T(), x.handle()), "exp"); }

// Sum / Mean / Max (full reductions, the tensor read as a flat vector)
template <class T, int... D> T sum(const Tensor<T, D...>& v) { return detail::sum(T(), v.handle()); }
template <class T, int... D> T mean(const Tensor<T, D...>& v) { return detail::mean(T(), v.handle()); }
template <class T, int... D> T max_of(const Tensor<T, D...>& v) { return detail::max(T(), v.handle()); }

}  // namespace cleave_cuda
