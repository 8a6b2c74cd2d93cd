// Plan object and the two label-form executors shared by tfb_execute and the einsum tree.
#pragma once
#include "common.h"

struct tfb_plan {
    tfb_ctx* ctx = nullptr;
    int dtype = TFB_F64;
    int op = 0;
    bool binary = false;
    int reduce_op = TFB_REDUCE_SUM;
    int force_kernel = 0;  // tfb::ContractKernel
    int algebra = 0;       // tfb_algebra
    std::vector<uint32_t> la, lb, lc;          // labels after lowering the descriptor
    std::vector<std::vector<int64_t>> shapes;  // inputs first, then output
    const char* kernel_name = "none";
};

namespace tfb {

tfb_status run_unary(tfb_ctx* ctx, int dtype, const std::vector<uint32_t>& labels_in, const HView& in,
                     const std::vector<uint32_t>& labels_out, const HView& out, Scalar alpha, Scalar beta,
                     int reduce_op, const char** used);

// With `d` the summed product is multiplied element-wise by d (labels a subset of the output's)
// before alpha and beta apply: c = alpha * (a b) . d + beta * c.
tfb_status run_binary(tfb_ctx* ctx, int dtype, const std::vector<uint32_t>& labels_a, const HView& a,
                      const std::vector<uint32_t>& labels_b, const HView& b, const std::vector<uint32_t>& labels_c,
                      const HView& c, Scalar alpha, Scalar beta, int force_kernel, const char** used,
                      const std::vector<uint32_t>* labels_d = nullptr, const HView* d = nullptr, int algebra = 0);

}  // namespace tfb
