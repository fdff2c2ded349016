// The reference's known-answer tests for the tensor path, written against the C++ host mirror
// (include/cleave_cuda.hpp) the way the reference writes them against its own stdlib:
//   cleave/tests/mlir_lower.rs:2034-2049 (vector add), :2077-2089 (matmul 2x3 . 3x2), :2098-2110 (matrix add),
//   :2135-2148 (rank-3 index), :2161-2184 (filled tensors), :2386-2433 (activations), :2441-2451 (sum / mean / max),
//   :2846-2858 (matmul with zero).
// Exit code 0 = all answers reproduced; prints the first mismatch otherwise.  Needs a CUDA device to run.
#include <cmath>
#include <cstdio>

#include "cleave_cuda.hpp"

using namespace cleave_cuda;

static int failures = 0;
#define EXPECT(cond)                                                     \
  do {                                                                   \
    if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); ++failures; } \
  } while (0)

template <class T>
static void run() {
  // vector add -> 11, 22, 33
  Tensor<T, 3> va{1, 2, 3}, vb{10, 20, 30};
  auto vc = va + vb;
  EXPECT(vc.at(0) == T(11) && vc.at(1) == T(22) && vc.at(2) == T(33));
  // matmul 2x3 . 3x2 -> 58, 64, 139, 154
  Tensor<T, 2, 3> ma{1, 2, 3, 4, 5, 6};
  Tensor<T, 3, 2> mb{7, 8, 9, 10, 11, 12};
  Tensor<T, 2, 2> mc = matmul(ma, mb);
  EXPECT(mc.at(0, 0) == T(58) && mc.at(0, 1) == T(64) && mc.at(1, 0) == T(139) && mc.at(1, 1) == T(154));
  // matrix add: c[0,0] = 11, c[1,1] = 44
  Tensor<T, 2, 2> a2{1, 2, 3, 4}, b2{10, 20, 30, 40};
  auto c2 = a2 + b2;
  EXPECT(c2.at(0, 0) == T(11) && c2.at(1, 1) == T(44));
  // the other ring operations
  auto d2 = (b2 - a2) * a2 / a2;
  EXPECT(d2.at(1, 0) == T(27));
  EXPECT((-a2).at(0, 1) == T(-2));
  // rank-3 construct + index
  Tensor<T, 2, 2, 2> r3{1, 2, 3, 4, 5, 6, 7, 8};
  EXPECT(r3.at(0, 1, 0) == T(3) && r3.at(1, 1, 1) == T(8));
  // filled tensors
  auto f7 = Tensor<T, 4, 5>::filled(T(7));
  EXPECT(f7.at(0, 0) == T(7) && f7.at(3, 4) == T(7));
  // matmul(a, zero) is exactly zero
  auto z = matmul(ma, Tensor<T, 3, 2>::zero());
  EXPECT(z.at(0, 0) == T(0) && z.at(1, 1) == T(0) && sum(z) == T(0));
  // activations: relu(-2) = 0, relu(3) = 3, sigmoid(0) = 0.5, tanh(0) = 0
  Tensor<T, 3> x{-2, 3, 0};
  auto r = relu(x);
  EXPECT(r.at(0) == T(0) && r.at(1) == T(3));
  EXPECT(sigmoid(x).at(2) == T(0.5) && tanh(x).at(2) == T(0) && exp(x).at(2) == T(1));
  // sum / mean / max of [1, 5, 3] = 9, 3, 5
  Tensor<T, 3> v{1, 5, 3};
  EXPECT(sum(v) == T(9) && mean(v) == T(3) && max_of(v) == T(5));
  // neuron forward (examples/neuron_demo.cleave:13-19): sigmoid(w . x + b) = 0.450166
  Tensor<T, 1, 3> w{T(0.5), T(-0.6), T(0.1)};
  Tensor<T, 3, 1> in{T(1.0), T(2.0), T(3.0)};
  auto pre = matmul(w, in) + Tensor<T, 1, 1>{T(0.2)};
  EXPECT(std::fabs(double(sigmoid(pre).at(0, 0)) - 0.450166) < 1e-6);
}

int main() {
  if (cleave_cuda_init(0) != 0) {
    std::printf("no device: %s\n", cleave_cuda_last_error_message());
    return 2;
  }
  try {
    run<float>();
    run<double>();
    // a length mismatch is an error, not a crash
    bool threw = false;
    try { Tensor<float, 4> bad(std::vector<float>(3, 0.f)); } catch (const Error& e) { threw = e.code == CLEAVE_CUDA_ERR_SHAPE; }
    EXPECT(threw);
  } catch (const Error& e) {
    std::printf("cleave_cuda::Error %d: %s\n", e.code, e.what());
    return 1;
  }
  if (failures == 0) std::printf("OK\n");
  return failures ? 1 : 0;
}
