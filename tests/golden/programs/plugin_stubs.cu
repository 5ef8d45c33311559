// Stand-ins for the three transform launchers of the reference's kernels/function.cu when a compiled
// program's generated code is built into a kernel plugin here.  function.cu itself needs CUDA 13
// (five-argument cudaGraphAddDependencies) and this image has CUDA 12.9; the generated
// function_map.cu takes the launchers' addresses for its ntt / int / sud records, so the symbols must
// exist - but they are never called: those records are served by libcerium_b200.so through the plugin
// shim, which keeps only the generated launchers of the OTHER record types.  TEST INFRASTRUCTURE.
#include <stdexcept>

#include "fhe.cuh"
#include "function.cuh"

namespace Cerium {
namespace __FNAME__ {

__host__ void _function_ntt_(cudaStream_t &, LimbDataType **, const LimbDataType **, const uint32_t *, const size_t,
                             const LimbDataType *, const LimbDataType2 *) {
  throw std::runtime_error("_function_ntt_: the reference transform launcher is not part of this plugin build");
}
__host__ void _function_sud_(cudaStream_t &, LimbDataType **, const LimbDataType **, const uint32_t *, const size_t,
                             const LimbDataType *, const LimbDataType2 *, const LimbDataType *, const LimbDataType *,
                             const uint32_t *) {
  throw std::runtime_error("_function_sud_: the reference transform launcher is not part of this plugin build");
}
__host__ void _function_int_(cudaStream_t &, LimbDataType **, const LimbDataType **, const uint32_t *, const size_t,
                             const LimbDataType *, const LimbDataType2 *) {
  throw std::runtime_error("_function_int_: the reference transform launcher is not part of this plugin build");
}

}  // namespace __FNAME__
}  // namespace Cerium
