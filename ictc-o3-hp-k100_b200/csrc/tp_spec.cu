// One translation unit per tensor-product spec: compile with -DICTC_SPEC=L222 (etc.).
#include "tp_tma_kernels.cuh"

#ifndef ICTC_SPEC
#error "compile with -DICTC_SPEC=<spec name from generated/tp_spec_tables.cuh>"
#endif

#define ICTC_CAT_(a, b) a##b
#define ICTC_CAT(a, b) ICTC_CAT_(a, b)
#define ICTC_DEFINE_(S) ICTC_TP_DEFINE(S)
#define ICTC_FAST_DEFINE_(S) ICTC_TP_FAST_DEFINE(S)
#define ICTC_ID_(S) ICTC_TP_##S##_ID
#define ICTC_ID(S) ICTC_ID_(S)

namespace ictc {
ICTC_DEFINE_(ICTC_SPEC)
ICTC_FAST_DEFINE_(ICTC_SPEC)
TpOps ICTC_CAT(tp_ops_, ICTC_SPEC)() { return make_ops_tma<TpSpec<ICTC_ID(ICTC_SPEC)>, ICTC_ID(ICTC_SPEC)>(); }
}  // namespace ictc
