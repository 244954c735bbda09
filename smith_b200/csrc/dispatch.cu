// dispatch.cu -- which kernel serves which shape.
#include "kernels.h"

namespace smith {

constexpr int kGemvMaxAutoRows = 4;  // measured: the dp4a kernel leads the mma.sync kernel up to four rows

// Small M is the decode regime (bound by streaming the packed weights once):
// the dp4a GEMV kernel for up to four rows, the integer mma.sync kernel up to
// 32.  Above that the tensor-core kernel takes over.  The any-shape kernel
// catches whatever the streaming kernels decline (odd N, ragged K, tiny problems).
int resolve_path(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (M <= kGemvMaxAutoRows && qgemv_supports(kind, M, N, K, groups)) return kGemv;
  if (M <= 32 && qdecode_supports(kind, M, N, K, groups)) return kDecode;
  if (qgemm_tc_supports(kind, M, N, K, groups)) return kTensor;
  return kGeneric;
}

}  // namespace smith
