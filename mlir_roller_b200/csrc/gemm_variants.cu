// Instantiates the tcgen05 GEMM kernel family: one kernel per buildable rTile and mode.
// The reference compiles a kernel per hint at run time (src/roller.py:358-387); here the set
// is fixed at build time and the search is told which tiles exist.
#include "gemm_variant_make.cuh"

namespace rb200 {

static const KernelVariant* table(int* n) {
  static const KernelVariant kTable[] = {
      make_variant<256, 1, 2>(), make_variant<256, 3, 2>(),
      make_variant<128, 1, 2>(), make_variant<128, 3, 2>(),
      make_variant<64, 1, 2>(),  make_variant<64, 3, 2>(),
      make_variant<256, 1, 1>(), make_variant<256, 3, 1>(),
      make_variant<128, 1, 1>(), make_variant<128, 3, 1>(),
      make_variant<64, 1, 1>(),  make_variant<64, 3, 1>(),
      // B given transposed (Bt[N,K]): both operands K-major
      make_variant<256, 1, 2, 1>(), make_variant<256, 3, 2, 1>(),
      make_variant<128, 1, 1, 1>(), make_variant<128, 3, 1, 1>(),
      make_variant<64, 1, 1, 1>(),  make_variant<64, 3, 1, 1>(),
      // skinny C (few rows): roles swapped, tile = 64 or 32 rows of C x 128 columns
      make_variant<64, 1, 1, 2>(),  make_variant<64, 3, 1, 2>(),
      make_variant<32, 1, 1, 2>(),  make_variant<32, 3, 1, 2>(),
  };
  *n = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));
  return kTable;
}

// Kernels whose ring fills shared memory, compiled a second time with one stage less and the
// staging area of the TMA-store output path.
static const KernelVariant* staged_table(int* n) {
  static const KernelVariant kTable[] = {
      make_variant<256, 1, 2, 0, 0, 1>(),
      make_variant<128, 1, 1, 0, 0, 1>(),
  };
  *n = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));
  return kTable;
}

const KernelVariant* find_staged_form(const KernelVariant* kv) {
  if (!kv || kv->staging_bytes > 0 || kv->gave_up_stage) return nullptr;
  int n;
  const KernelVariant* t = (kv->mode == 16 || kv->mode == 17) ? staged_forms_16bit(&n)
                                                             : staged_table(&n);
  for (int i = 0; i < n; ++i) {
    if (t[i].block_m == kv->block_m && t[i].block_n == kv->block_n && t[i].rstep == kv->rstep &&
        t[i].cta_group == kv->cta_group && t[i].mode == kv->mode && t[i].layout == kv->layout)
      return &t[i];
  }
  return nullptr;
}

int variant_count() {
  int n;
  table(&n);
  return n;
}

const KernelVariant& variant_at(int idx) {
  int n;
  return table(&n)[idx];
}

const KernelVariant* find_variant(int block_m, int block_n, int rstep, int cta_group, int mode,
                                  int layout) {
  if (layout == 3) {
    const KernelVariant* v = simt_skinny_variant();
    return (v->block_m == block_m && v->block_n == block_n && v->rstep == rstep &&
            v->cta_group == cta_group && v->mode == mode) ? v : nullptr;
  }
  int n;
  const KernelVariant* t = (mode == 16 || mode == 17) ? variants_16bit(&n) : table(&n);
  for (int i = 0; i < n; ++i) {
    if (t[i].block_m == block_m && t[i].block_n == block_n && t[i].rstep == rstep &&
        t[i].cta_group == cta_group && t[i].mode == mode && t[i].layout == layout)
      return &t[i];
  }
  return nullptr;
}

}  // namespace rb200
