// Translation unit of the engine's code object: every sm_100a kernel of the routed-MoE path,
// compiled to netra_moe_sm100a.cubin and loaded by the engine runtime through the driver API.
#include "bridge_kernels.cu"
#include "route_kernels.cu"
#include "umma_kernels.cu"
#include "umma_tokmajor.cu"
#include "router_umma.cu"
