// double-compute instantiation of the element-wise family.
#include "elementwise_impl.cuh"
namespace b200ew {
int dispatch_f64(const B200EwDesc& d, cudaStream_t s) { return dispatch<double>(d, s); }
}
