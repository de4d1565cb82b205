// Instantiations of the projection kernel for one weight kind (its own translation unit so the kinds compile in
// parallel). See linear.cu for the design and linear_kernel.cuh for the kernel.
#include "linear_kernel.cuh"

namespace b200dec_detail {

int launch_24(const LinArgs& a, bool split, bool ln, int warps, int k, int ksplit, bool pdl, cudaStream_t s) {
  if (split) return fail(B200DEC_EINVAL, "linear: 2:4 weights take the fp16 operand");
  return ln ? launch_shape<B200DEC_W_INT8_24, false, true>(a, warps, k, ksplit, pdl, s)
            : launch_shape<B200DEC_W_INT8_24, false, false>(a, warps, k, ksplit, pdl, s);
}

bool fits_24(bool split, bool ln, int warps, int k, int ksplit, int rows) {
  if (split) return false;
  return ln ? fits_shape<B200DEC_W_INT8_24, false, true>(warps, k, ksplit, rows) : fits_shape<B200DEC_W_INT8_24, false, false>(warps, k, ksplit, rows);
}

}  // namespace b200dec_detail
