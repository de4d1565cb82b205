// Instantiations of the projection kernel for one weight kind (its own translation unit so the kinds compile in
// parallel). See linear.cu for the design and linear_kernel.cuh for the kernel.
#include "linear_kernel.cuh"

namespace b200dec_detail {

int launch_f16(const LinArgs& a, bool split, int ln, int warps, int k, int ksplit, bool pdl, cudaStream_t s) {
  if (split) {
    if (ln == 2) return fail(B200DEC_EINVAL, "linear: fp16 LayerNorm rows go with the single fp16 operand");
    return ln ? launch_shape<B200DEC_W_F16, true, 1>(a, warps, k, ksplit, pdl, s)
              : launch_shape<B200DEC_W_F16, true, 0>(a, warps, k, ksplit, pdl, s);
  }
  if (ln == 2) return launch_shape<B200DEC_W_F16, false, 2>(a, warps, k, ksplit, pdl, s);
  return ln ? launch_shape<B200DEC_W_F16, false, 1>(a, warps, k, ksplit, pdl, s)
            : launch_shape<B200DEC_W_F16, false, 0>(a, warps, k, ksplit, pdl, s);
}

bool fits_f16(bool split, int ln, int warps, int k, int ksplit, int rows) {
  if (split) return ln == 2 ? false : ln ? fits_shape<B200DEC_W_F16, true, 1>(warps, k, ksplit, rows) : fits_shape<B200DEC_W_F16, true, 0>(warps, k, ksplit, rows);
  if (ln == 2) return fits_shape<B200DEC_W_F16, false, 2>(warps, k, ksplit, rows);
  return ln ? fits_shape<B200DEC_W_F16, false, 1>(warps, k, ksplit, rows) : fits_shape<B200DEC_W_F16, false, 0>(warps, k, ksplit, rows);
}

}  // namespace b200dec_detail
