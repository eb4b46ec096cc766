// Kernels of the local sort for 1-byte keys.
#include "b2s_launch.cuh"
namespace b2s {
B2S_INSTANTIATE_KEY_WIDTH(1, false, false)
}
