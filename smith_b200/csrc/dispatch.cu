// dispatch.cu -- which kernel serves which shape.
#include "kernels.h"

namespace smith {

// M <= 16 is the decode regime (bound by streaming the packed weights once);
// above that the tensor-core kernel takes over; the any-shape kernel catches
// whatever the two streaming kernels decline (odd N, ragged K, tiny problems).
int resolve_path(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (M <= 16 && qdecode_supports(kind, M, N, K, groups)) return kDecode;
  if (M > 16 && qgemm_tc_supports(kind, M, N, K, groups)) return kTensor;
  return kGeneric;
}

}  // namespace smith
