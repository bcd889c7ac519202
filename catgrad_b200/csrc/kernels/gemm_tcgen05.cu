// placeholder while the tensor-core kernel is being written
#include "gemm_tcgen05.h"
namespace cgk {
bool tcgen05_gemm_applicable(const View4&, long long, const void*, const void*, long long, long long, long long,
                             long long, long long, long long, long long) { return false; }
void launch_tcgen05_gemm(const View4&, long long, const void*, const void*, void*, long long, long long, long long,
                         long long, long long, unsigned*, int, cudaStream_t) {}
}
