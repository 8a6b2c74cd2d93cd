// Device-resident offset tables of one normalised contraction layout, cached per
// (device, layout) so that a loop over the same einsum builds them once.
#pragma once
#include "common.h"
#include "contract_common.cuh"

namespace tfb {

struct ContractTables {
    void* block = nullptr;
    int64_t *a_b = nullptr, *b_b = nullptr, *c_b = nullptr;
    int64_t *a_m = nullptr, *c_m = nullptr, *b_n = nullptr, *c_n = nullptr, *a_k = nullptr, *b_k = nullptr;
    int64_t *d_b = nullptr, *d_m = nullptr, *d_n = nullptr;  // the fused multiplier's offsets, when the problem has one
    int64_t M = 0, N = 0, K = 0, B = 0;
    // The tables are filled by kernels on the stream of whichever context missed the cache
    // first.  `built` is recorded behind those kernels; a later user on another stream waits
    // for it (get_tables does), `ready` remembers that the event has been seen complete.
    cudaEvent_t built = nullptr;
    cudaStream_t build_stream = nullptr;
    bool ready = false;
    ~ContractTables();
};

tfb_status get_tables(tfb_ctx* ctx, const ContractProblem& p, std::shared_ptr<ContractTables>* out);
void fill_args(const ContractProblem& p, const ContractTables& t, ContractArgs* a);

}  // namespace tfb
