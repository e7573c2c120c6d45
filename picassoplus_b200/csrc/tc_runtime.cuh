// Host-side state shared by the three tensor-core kernels of facet2facet: the operand
// format a precision mode stands for, the per-device word a kernel raises when one of its
// bounded waits ran out, and the wait budget handed to every launch.
#pragma once
#include "common.cuh"

namespace pb {
namespace tc {

// precision mode -> operand splits (1, or 2 = hi + lo with three products per term) and
// operand format (bf16, else tf32)
struct OperandMode { int nsplit, bf; };
inline OperandMode operand_mode(int precision) {
    OperandMode m;
    m.nsplit = (precision == PB200_PREC_FP32 || precision == PB200_PREC_FP32_TF32X3) ? 2 : 1;
    m.bf = (precision == PB200_PREC_BF16 || precision == PB200_PREC_FP32) ? 1 : 0;
    return m;
}

// Mapped, pinned host word of the current device (0 = no kernel gave up); nullptr if the
// one-time allocation failed.  The first call allocates (outside stream capture).
int* async_error_word();
// PB200_ECUDA (with error text) if a tensor-core kernel on the current device gave up since
// the last pb200_clear_async_error()
int check_async_error(const char* where);

// wait budget of the next launches in units of 1024 clocks, and the test switch that makes
// the forward kernel's filter stream stay silent (so that its waits run out)
int wait_budget_kclocks();
int test_skip_filter_stream();

}  // namespace tc
}  // namespace pb
