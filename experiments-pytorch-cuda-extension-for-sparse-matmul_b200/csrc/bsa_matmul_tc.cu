#include "bsa_common.cuh"
namespace bsa {
bool tc_supports(const MatmulArgs&) { return false; }
int matmul_tc(const MatmulArgs&) { return BSA_ERR_BAD_SHAPE; }
}
