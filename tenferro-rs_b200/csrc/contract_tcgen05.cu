// f32 / Complex32 contraction on the 5th-generation tensor cores (placeholder: declines).
#include "common.h"
namespace tfb {
tfb_status contract_tcgen05(tfb_ctx*, const ContractProblem&, bool* declined) {
    *declined = true;
    return TFB_OK;
}
}  // namespace tfb
