// Operand of the tensor-core matrix multiply as it lies in memory (shared by gemm_tc.cu, conv.cu).
#pragma once
namespace b200 {
// `rows` x `cols` row-major with pitch `ld`; p1 is the TF32 tail when the operand was split
// (3xTF32), else unused. shared = one matrix for every batch entry.
struct TcOperand {
  const void *p0 = nullptr, *p1 = nullptr;
  long long ld = 0, batch_stride = 0;
  bool shared = false;
};
}  // namespace b200
