// Builds the softmax drivers' own gold functions (cpu_softmax, cpu_logsoftmax of
// test/softmax_test_common.c.inc in the FStarLang/kuiper tree) into the reference CPU library.
// The include's test runner wants a kernel to call; it gets a stub, nothing here runs on a GPU.
// Compile with: -I <kuiper>/include -I <kuiper>/test
#include <stdint.h>
#define SCALAR double
#define TO_DOUBLE(x) (x)
#define FROM_DOUBLE(x) (x)
#define FUN(lena, a) ((void)(lena), (void)(a))
#define FUN_N(nth, lena, a) ((void)(nth), (void)(lena), (void)(a))
#define LABEL "unused"
#define ATOL 0.0
#define RTOL 0.0
#define IS_LOGSOFTMAX 0
namespace ref_softmax_ns {
#include "softmax_test_common.c.inc"
}
extern "C" void ref_cpu_softmax(const double *in, double *out, int n) { ref_softmax_ns::cpu_softmax(in, out, n); }
extern "C" void ref_cpu_logsoftmax(const double *in, double *out, int n) { ref_softmax_ns::cpu_logsoftmax(in, out, n); }
