// Finite-field constants, element types and operator codes of the muGraph
// executor.  Names and numeric values are those of the reference
// (include/mirage/type.h:26-129) because they are part of its API and of the
// bit-exact fingerprint contract; everything else in this tree is new code.
#pragma once
#include <cassert>
#include <cstddef>
#include <cstdint>

namespace mirage {
namespace type {

// Fingerprints are stored as 16-bit values < FP_PQ and combined in 32/64-bit integers.
using FPType = uint16_t;
constexpr uint16_t FP_P = 227, FP_Q = 113, FP_PQ = 25651;
constexpr uint32_t FP_EXP_BASE = 3;
constexpr uint16_t FP_P_MUL_Q_MOD_1 = 227;   // multiple of P, congruent to 1 mod Q
constexpr uint16_t FP_Q_MUL_P_MOD_1 = 25425; // multiple of Q, congruent to 1 mod P

// Shared memory a threadblock graph may plan.  The reference stops at 96 KB; sm_100 offers
// 227 KB of dynamic shared memory per block and the dense attention tiles need it.
constexpr size_t MAX_SMEM_SIZE = 227 * 1024;
constexpr int TB_REDUCTION_DIMX = 64;

enum DataType { DT_INT8 = 900, DT_UINT16 = 910, DT_BFLOAT16 = 920, DT_FLOAT16 = 921, DT_FLOAT32 = 930,
                DT_DOUBLE = 940, DT_UNKNOWN = 999 };
size_t get_datatype_size(DataType type);

enum KNOperatorType { KN_UNKOWN = 1000, KN_INPUT_OP = 1001, KN_MATMUL_OP = 1003, KN_REDUCTION_0_OP = 1004,
                      KN_REDUCTION_1_OP = 1005, KN_REDUCTION_2_OP = 1006, KN_EXP_OP = 1007, KN_ADD_OP = 1008,
                      KN_MUL_OP = 1009, KN_DIV_OP = 1010, KN_CUSTOMIZED_OP = 1999 };

enum TBOperatorType { TB_UNKOWN = 2000, TB_INPUT_OP = 2001, TB_OUTPUT_OP = 2002, TB_MATMUL_OP = 2003,
                      TB_EXP_OP = 2007, TB_ADD_OP = 2008, TB_MUL_OP = 2009, TB_DIV_OP = 2010,
                      TB_CONCAT_THEN_MATMUL_OP = 2011,
                      TB_REDUCTION_FIRST_OP_ID = 2100, TB_REDUCTION_0_OP = 2101, TB_REDUCTION_1_OP = 2102,
                      TB_REDUCTION_2_OP = 2103, TB_REDUCTION_0_TO_DIMX_OP = 2104, TB_REDUCTION_1_TO_DIMX_OP = 2105,
                      TB_REDUCTION_2_TO_DIMX_OP = 2106, TB_REDUCTION_LAST_OP_ID = 2199,
                      TB_CONCAT_FIRST_OP_ID = 2200, TB_CONCAT_0_OP = 2200, TB_CONCAT_1_OP = 2201,
                      TB_CONCAT_2_OP = 2202, TB_CONCAT_LAST_OP_ID = 2210, TB_CUSTOMIZED_OP = 2999 };

enum ActivationType { ACT_UNKOWN = 3000, ACT_EXP = 3001, ACT_RELU = 3002, ACT_GELU = 3003, ACT_NONE = 3100 };

// JSON names used by the reference's graph wire format (type.h:64-129)
char const *to_string(KNOperatorType t);
char const *to_string(TBOperatorType t);

} // namespace type
} // namespace mirage
