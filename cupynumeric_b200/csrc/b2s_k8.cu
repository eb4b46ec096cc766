// Kernels of the local sort for 8-byte keys.
#include "b2s_launch.cuh"
namespace b2s {
B2S_INSTANTIATE_KEY_WIDTH(8, true, true)
}
