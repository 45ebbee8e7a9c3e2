#include "tensor_path.cuh"
namespace pcb {
bool tensor_path_supported(Pass, int, int, const Geom&) { return false; }
size_t tensor_scratch_bytes(Pass, int, int, int, const Geom&) { return 0; }
int tensor_launch(Pass, int, int, const Geom&, const void*, const void*, const void*, void*, float*, int*, cudaStream_t) { return PCB_ERR_UNSUPPORTED; }
}
