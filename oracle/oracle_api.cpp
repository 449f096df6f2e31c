// ORACLE -- test infrastructure, not product code.
// C entry points (`orc_*`) over the CPU restatement in cpu_backend.hpp, with the
// same shape as the CUDA library's `rth_*` engine API so that a test can run one
// graph on both and compare.  Built by oracle/Makefile into oracle/liboracle.so.
#include "cpu_backend.hpp"
#include "../rusttensor_b200/csrc/host/engine_capi.hpp"

RT_DEFINE_ENGINE_CAPI(orc, oracle::CpuBackend)

extern "C" {
// 1 (default): reproduce the reference's conv2d input-gradient defect
// (src/ops/cpu_ops.rs:266,271).  0: mathematically correct col2im.
void orc_set_conv_dx_faithful(int on) { oracle::conv_dx_faithful() = on != 0; }
int orc_get_conv_dx_faithful() { return oracle::conv_dx_faithful() ? 1 : 0; }
}
