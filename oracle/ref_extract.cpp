// Build-time helper (test infrastructure): prints the OpenCL C source string the
// reference keeps in src/backend/generic/runtime/opencl/kernels.h, so that
// oracle/Makefile can compile the reference's own kernel bodies as plain C.
// The text is read from the reference tree where it lies and written only under
// oracle/_ref/, which is not tracked.
#include REF_KERNELS_H
#include <cstdio>
int main() {
  std::fwrite(textKernels.data(), 1, textKernels.size(), stdout);
  return 0;
}
