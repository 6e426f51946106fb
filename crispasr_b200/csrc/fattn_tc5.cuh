// fattn_tc5.cuh — interface of the TMA + tcgen05 + TMEM prefill kernel (fattn_tc5.cu).
#pragma once
#include "fattn_common.cuh"

namespace b200 {

// True when the operands fit the tcgen05 kernels: F16 K/V with 16-byte aligned strides, head_dim 64 or 128 (128
// for the fused rel-pos form), no softcap/ALiBi; explicit F16 masks, the implicit causal mask and kv_len are
// handled in-kernel.
bool tc5_supported(const FattnArgs& a);

// Encodes the tensor maps and launches. Returns a B200_* code; on CUDA failure writes the text to errbuf.
int launch_prefill_tc5(const FattnArgs& a, cudaStream_t st, char* errbuf, size_t errlen);

// Reads the device status word set when a bounded device-side wait ran out (0 = never). Returns a cudaError_t value.
int tc5_read_status(int* status);
int tc5_reset_status();

}  // namespace b200
