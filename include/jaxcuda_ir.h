/*
 * Wire format of a lowered Kernel, as handed to jaxcuda_prepare_kernel().
 *
 * The image is what the reference's TypeScript side holds after
 * `tuneNullopt`-style lowering (src/tuner.ts:219-240): gidx/ridx bound to
 * ranged Specials, GlobalView rewritten to Where(valid, GlobalIndex, 0)
 * (src/alu.ts:1664-1679), the body cast to the accumulator dtype.  Node
 * fields are the four fields of `AluExp` (src/alu.ts:138-143); the header is
 * `Kernel` (src/alu.ts:1479-1527) plus `Reduction` (src/alu.ts:1544-1569).
 *
 * All words are little-endian uint32.
 *
 *   word 0      JAXCUDA_IR_MAGIC
 *   word 1      nargs          number of input buffers
 *   word 2,3    size           output element count (lo, hi)
 *   word 4      has_reduction  0 | 1
 *   word 5      reduction dtype   (jaxcuda_dtype; accumulator type)
 *   word 6      reduction op      (JAXCUDA_OP_ADD | MUL | MIN | MAX)
 *   word 7      reduction size    K, the trip count of ridx
 *   word 8      n_exp          nodes of the body, topologically ordered, root last
 *   word 9      n_epi          nodes of the epilogue (0 without a reduction)
 *   then (n_exp + n_epi) nodes of JAXCUDA_IR_NODE_WORDS words each:
 *     +0 op   +1 dtype   +2 nsrc   +3..+6 src[4] (indices into the same list)
 *     +7,+8 arg0 (64 bit)   +9 arg1
 *
 *   arg0/arg1 by op:
 *     Const        arg0 = IEEE double bits (float dtypes) or two's-complement int64
 *     Special      arg0 = 0 gidx | 1 ridx, arg1 = n (index range is [0, n))
 *     Variable     arg0 = 0 ("acc", epilogue only)
 *     GlobalIndex  arg0 = gid (input buffer number), arg1 = len (elements); src[0] = int32 index
 *     BitCombine   arg0 = 0 and | 1 or | 2 xor
 *     BitShift     arg0 = 0 shl | 1 shr
 *     Threefry2x32 arg0 = 0 xor of both words | 1 first word | 2 second word
 */
#ifndef JAXCUDA_IR_H
#define JAXCUDA_IR_H

#include <stdint.h>

#define JAXCUDA_IR_MAGIC 0x314B584Au /* "JXK1" */
#define JAXCUDA_IR_HEADER_WORDS 10
#define JAXCUDA_IR_NODE_WORDS 10

/* src/alu.ts:6-13.  Bool occupies 4 bytes holding 0 or 1 (alu.ts:23-29, :95). */
typedef enum {
  JAXCUDA_F32 = 0,
  JAXCUDA_I32 = 1,
  JAXCUDA_U32 = 2,
  JAXCUDA_BOOL = 3,
  JAXCUDA_F16 = 4,
  JAXCUDA_F64 = 5
} jaxcuda_dtype;

/* src/alu.ts:1365-1407, in declaration order. */
typedef enum {
  JAXCUDA_OP_ADD = 0, JAXCUDA_OP_SUB, JAXCUDA_OP_MUL, JAXCUDA_OP_IDIV, JAXCUDA_OP_MOD,
  JAXCUDA_OP_MIN, JAXCUDA_OP_MAX,
  JAXCUDA_OP_SIN, JAXCUDA_OP_COS, JAXCUDA_OP_ASIN, JAXCUDA_OP_ATAN, JAXCUDA_OP_EXP,
  JAXCUDA_OP_LOG, JAXCUDA_OP_ERF, JAXCUDA_OP_ERFC, JAXCUDA_OP_SQRT, JAXCUDA_OP_FLOOR,
  JAXCUDA_OP_CEIL, JAXCUDA_OP_RECIPROCAL, JAXCUDA_OP_CAST, JAXCUDA_OP_BITCAST,
  JAXCUDA_OP_BITCOMBINE, JAXCUDA_OP_BITINVERT, JAXCUDA_OP_BITSHIFT,
  JAXCUDA_OP_CMPLT, JAXCUDA_OP_CMPNE, JAXCUDA_OP_WHERE, JAXCUDA_OP_THREEFRY2X32,
  JAXCUDA_OP_CONST, JAXCUDA_OP_SPECIAL, JAXCUDA_OP_VARIABLE, JAXCUDA_OP_GLOBALINDEX,
  JAXCUDA_OP_COUNT
} jaxcuda_op;

#endif /* JAXCUDA_IR_H */
