// What each TMA / tcgen05 kernel of the library allocates per block: the figures Gern's
// Allocates(reg, smem) statement (include/gern/annotations/stmt.h:113-121) would carry, taken from
// the kernels' planned layouts (smem_plan.hpp) instead of being stated by hand.  The host layer
// checks a program's Global(..., smem_size) and its pinned cluster dimension against them.
#include <string.h>

#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {
int kernel_regs_gemm_tc();
int kernel_regs_gemm_2cta();
int kernel_regs_attention();
int kernel_regs_attention_pair();
}  // namespace gb200

using namespace gb200;

extern "C" int gb200_kernel_resources_query(const char *kernel, gb200_kernel_resources *out) {
    GB200_REQUIRE(kernel != nullptr && out != nullptr, GB200_ERR_INVALID_ARG, "NULL argument");
    memset(out, 0, sizeof(*out));
    if (strcmp(kernel, "gemm_bf16_tc") == 0) {
        constexpr smem::GemmTcLayout l = smem::gemm_tc_layout(256);
        *out = {kernel_regs_gemm_tc(), smem::GemmTcLayout::kThreads, l.dynamic_bytes, smem::GemmTcLayout::kCluster,
                smem::GemmTcLayout::kTmemColumns};
    } else if (strcmp(kernel, "gemm_bf16_2cta") == 0) {
        constexpr smem::Gemm2CtaLayout l = smem::gemm_2cta_layout(6);
        *out = {kernel_regs_gemm_2cta(), smem::Gemm2CtaLayout::kThreads, l.dynamic_bytes, smem::Gemm2CtaLayout::kCluster,
                smem::Gemm2CtaLayout::kTmemColumns};
    } else if (strcmp(kernel, "attention_bf16") == 0) {
        constexpr smem::AttentionLayout l = smem::attention_layout(320);
        *out = {kernel_regs_attention(), l.threads, l.dynamic_bytes, smem::AttentionLayout::kCluster,
                smem::AttentionLayout::kTmemColumns};
    } else if (strcmp(kernel, "attention_bf16_pair") == 0) {
        constexpr smem::AttentionPairLayout l = smem::attention_pair_layout();
        *out = {kernel_regs_attention_pair(), smem::AttentionPairLayout::kThreads, l.dynamic_bytes,
                smem::AttentionPairLayout::kCluster, smem::AttentionPairLayout::kTmemColumns};
    } else {
        set_error("no kernel named '%s' (known: gemm_bf16_tc, gemm_bf16_2cta, attention_bf16, attention_bf16_pair)",
                  kernel);
        return GB200_ERR_INVALID_ARG;
    }
    return GB200_OK;
}
