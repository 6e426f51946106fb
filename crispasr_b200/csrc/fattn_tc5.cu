#include "fattn_tc5.cuh"
namespace b200 {
bool tc5_supported(const FattnArgs&) { return false; }
int launch_prefill_tc5(const FattnArgs&, cudaStream_t, char*, size_t) { return B200_E_UNSUPPORTED; }
}
