// Decode projections with 4 tiles of 16 rows of x (up to 64 rows): the instantiations of
// gemv_kernel.cuh for that many tiles, in a file of their own so that the four files
// compile side by side.
#include "gemv_kernel.cuh"

namespace nnis {

int gemv_launch_tiles4(const GemvArgs& a, int epilogue, int prologue, const GemvPlan& plan, bool pdl,
                        cudaStream_t stream) {
    return launch_gemv_epi<4>(a, epilogue, prologue, plan, pdl, stream);
}

}  // namespace nnis
