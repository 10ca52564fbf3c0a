// The kernels for 16-bit operands (bf16 or fp16 A and B, fp32 C): the same template as the fp32
// family with tcgen05.mma kind::f16 and a reduce step of 64. The reference's problem
// descriptor is parametric in the element width (src/analyze.py:31,39-41) although its kernel
// generator only emits f32 (src/roller.py:47-68); these variants are what a 16-bit
// MatmulConfig binds to.
#include "gemm_variant_make.cuh"

namespace rb200 {

template <int DT>
static void fill(KernelVariant* out, int* n) {
  int i = 0;
  out[i++] = make_variant<256, 1, 2, 0, DT>();
  out[i++] = make_variant<128, 1, 2, 0, DT>();
  out[i++] = make_variant<256, 1, 1, 0, DT>();
  out[i++] = make_variant<128, 1, 1, 0, DT>();
  out[i++] = make_variant<64, 1, 1, 0, DT>();
  // B given transposed: both operands K-major
  out[i++] = make_variant<256, 1, 2, 1, DT>();
  out[i++] = make_variant<128, 1, 1, 1, DT>();
  out[i++] = make_variant<64, 1, 1, 1, DT>();
  // skinny C
  out[i++] = make_variant<64, 1, 1, 2, DT>();
  out[i++] = make_variant<32, 1, 1, 2, DT>();
  *n = i;
}

const KernelVariant* variants_16bit(int* n) {
  static KernelVariant kTable[32];
  static int count = [] {
    int a = 0, b = 0;
    fill<1>(kTable, &a);
    fill<2>(kTable + a, &b);
    return a + b;
  }();
  *n = count;
  return kTable;
}

const KernelVariant* staged_forms_16bit(int* n) {
  static const KernelVariant kTable[] = {
      make_variant<256, 1, 2, 0, 1, 1>(), make_variant<128, 1, 1, 0, 1, 1>(),
      make_variant<256, 1, 2, 0, 2, 1>(), make_variant<128, 1, 1, 0, 2, 1>(),
  };
  *n = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));
  return kTable;
}

}  // namespace rb200
