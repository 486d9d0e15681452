// Link shim of the kernels-only reference arm (bench.py --impl reference).
//
// The reference's CUDA translation units are compiled unmodified from the reference tree.  Two of them call the reference's
// PerfStatsCollector, whose implementation needs libfort (fetched over the network by the reference's CMake build and not
// available offline): the two entry points they use are defined here as "disabled".  The GPU repack launcher has C++
// linkage; a C wrapper makes it callable through ctypes.  Nothing else of the reference is replaced.
#include <cstdint>
#include <map>
#include <string>

#include "kernels/cuda/repack/CUDAVnniRepackKernels.h"
#include "utils/PerfStatsCollector.h"

namespace llaminar2 {
bool PerfStatsCollector::isEnabled() { return false; }
void PerfStatsCollector::addCounter(std::string, std::string, double, std::string, std::string, Tags) {}
}  // namespace llaminar2

extern "C" int ref_repack_to_vnni(int format, const void* d_raw, uint8_t* d_payload, uint16_t* d_scales, uint16_t* d_mins,
                                  int n, int k, void* stream) {
    return llaminar2::launchVnniRepackCUDA(static_cast<llaminar2::RepackFormat>(format), d_raw, d_payload, d_scales, d_mins, n, k, stream) ? 1 : 0;
}
