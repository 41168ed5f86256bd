// C entry point to the reference's own Q8_0 -> Q2_0 requantizer (arch/qwen4exp/mtp.hpp:40), for the
// parity tests. TEST INFRASTRUCTURE ONLY. Linked with the reference's arch/qwen4exp/mtp.cu compiled
// unmodified from the reference tree (see the Makefile); nothing of the reference is copied here.
#include <cstddef>
#include <cstdint>

namespace flashrt::qwen4exp {
void convert_q8_0_to_q2_0(const uint8_t* src, uint8_t* dst, size_t nblocks64, int threads);
}

extern "C" void ref_convert_q8_0_to_q2_0(const uint8_t* src, uint8_t* dst, size_t nblocks64, int threads) {
    flashrt::qwen4exp::convert_q8_0_to_q2_0(src, dst, nblocks64, threads);
}
