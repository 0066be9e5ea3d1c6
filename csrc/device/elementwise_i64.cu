// integer/bool-compute instantiation of the element-wise family.
#include "elementwise_impl.cuh"
namespace b200ew {
int dispatch_i64(const B200EwDesc& d, cudaStream_t s) { return dispatch<long long>(d, s); }
}
