#include "runtime.hpp"
namespace anl {
struct GemmPlan {};
int plan_gemm(anl_device*, const Item&, Plan&) { return ANL_ERR_UNSUPPORTED; }
int launch_gemm(anl_device* dev, const Plan&, void* const*, cudaStream_t) { return dev->fail(ANL_ERR_UNSUPPORTED, "gemm: not built"); }
}
