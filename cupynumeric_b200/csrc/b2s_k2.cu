// Kernels of the local sort for 2-byte keys.
#include "b2s_launch.cuh"
namespace b2s {
B2S_INSTANTIATE_KEY_WIDTH(2, true, false)
}
