// Source of the mangled symbols in function_base.tsv: compiled with g++ -c and listed with nm by make_golden.py.
// Shapes seen in real traces: namespaces, templates with non-type arguments, anonymous namespaces, lambdas passed as
// template arguments, enable_if expressions with comparison operators inside parentheses, operators.
#include <type_traits>
namespace at { namespace native {
template <int N, typename F, typename A> void vectorized_elementwise_kernel(int n, F f, A a) {}
template <typename T> struct Add { T operator()(T a, T b) const { return a + b; } };
template <typename T, int VEC> void reduce_kernel(T* out, const T* in, long n) {}
namespace { template <typename scalar_t> void cunn_SoftMaxForward(scalar_t* o, const scalar_t* i, int d) {} void plain_anonymous(float*) {} }
template <int A, int B> typename std::enable_if<((A) > (B)), void>::type cond_kernel(float*) {}
template <int A, int B> typename std::enable_if<(A < B), int>::type cond_kernel2(double*) { return 0; }
struct Functor { void operator()(int) const {} bool operator<(const Functor&) const { return false; } };
}}
namespace cutlass { template <typename Op> void Kernel(typename Op::Params p) {} struct Gemm { struct Params { int m; }; }; }
void sleep_kernel(int) {}
extern "C" void _apply_write_kernel(float*) {}
template <typename T> T templated_return(T x) { return x; }
template <typename... Ts> void variadic_kernel(Ts...) {}
void use() {
  at::native::vectorized_elementwise_kernel<4>(1, at::native::Add<float>(), 3);
  at::native::vectorized_elementwise_kernel<8>(1, [](float a) { return a; }, 2.0);
  at::native::reduce_kernel<float, 4>(nullptr, nullptr, 0);
  at::native::reduce_kernel<double, 1>(nullptr, nullptr, 0);
  at::native::cunn_SoftMaxForward<float>(nullptr, nullptr, 0);
  at::native::plain_anonymous(nullptr);
  at::native::cond_kernel<8, 0>(nullptr);
  at::native::cond_kernel2<1, 2>(nullptr);
  at::native::Functor f; f(1); (void)(f < f);
  cutlass::Kernel<cutlass::Gemm>({1});
  sleep_kernel(1);
  templated_return<int>(1);
  templated_return<at::native::Add<int>>({});
  variadic_kernel(1, 2.0f, 'c');
  variadic_kernel();
}
