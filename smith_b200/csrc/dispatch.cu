// dispatch.cu -- which kernel serves which shape.
#include "kernels.h"

namespace smith {

// measured: the dp4a kernel leads the mma.sync kernel up to three rows, and at four rows where the
// output is narrow (4096 x 4096: 9.8 us against 12.7 us; 4096 x 14336: 21.2 us against 17.3 us)
constexpr int kGemvMaxAutoRows = 4;

// Small M is the decode regime (bound by streaming the packed weights once):
// the dp4a GEMV kernel for up to four rows, the integer mma.sync kernel up to
// 16, and up to 32 where the output is narrow (measured: from 17 rows on the
// tcgen05 kernel leads once N fills its column tiles, 28 us against 38 us at
// 4096 x 14336, while at N = 4096 the mma.sync kernel keeps a small lead).
// Above that the tensor-core kernel takes over.  The any-shape kernel
// catches whatever the streaming kernels decline (odd N, ragged K, tiny problems).
int resolve_path(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  const bool four_wide = M == kGemvMaxAutoRows && N >= 8192 && qdecode_supports(kind, M, N, K, groups);
  if (M <= kGemvMaxAutoRows && !four_wide && qgemv_supports(kind, M, N, K, groups)) return kGemv;
  const bool wide = N >= 8192 && qgemm_tc_supports(kind, M, N, K, groups);
  if ((M <= 16 || (M <= 32 && !wide)) && qdecode_supports(kind, M, N, K, groups)) return kDecode;
  if (qgemm_tc_supports(kind, M, N, K, groups)) return kTensor;
  return kGeneric;
}

}  // namespace smith
