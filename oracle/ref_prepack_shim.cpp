// Build shim for the REFERENCE's own binary prepack (test infrastructure only).
// It compiles lowbit_kernel/csrc/utils/weight_prepacking.h where it lies in the reference checkout
// (include path given by the Makefile) and exports bin_matrix_prepacking_to_uint32 with C linkage.
// No reference source is copied here; the output goes to oracle/_ref/ which is never committed.
#include <cstdint>
#include <cstddef>
#include <cstring>
#include <cuda_fp16.h>
#include "lowbit_kernel/csrc/utils/weight_prepacking.h"

extern "C" void ref_bin_matrix_prepacking_to_uint32(uint32_t* packed, const uint16_t* fp16_rows, size_t M, size_t K) {
    // The reference ORs bits into a malloc'd buffer without clearing it (fp6_linear.cu:468); clear first.
    std::memset(packed, 0, M * K / 8);
    bin_matrix_prepacking_to_uint32(packed, reinterpret_cast<half*>(const_cast<uint16_t*>(fp16_rows)), M, K);
}
