// Element types and reductions shared by the host scheduler and the kernels.
#pragma once
#include <cstdint>

namespace chb {
enum DType : int32_t { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_I32 = 3, DT_F64 = 4, DT_I64 = 5, DT_U8 = 6 };
enum RedOp : int32_t { OP_SUM = 0, OP_MAX = 1, OP_MIN = 2, OP_PROD = 3 };
int dtype_size(int dt);
}  // namespace chb
