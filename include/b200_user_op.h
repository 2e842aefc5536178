/* Calling convention of a user-written CUDA op that `make_torch_op_from_mojo` turns into a torch
 * custom op and that a graph compiled with `mojo_backend` launches without a graph break.
 *
 * Replaces, for CUDA sources, the reference's registration of user kernels written in Mojo
 * (torch_mojo_backend/custom_torch_ops_in_mojo/torch_custom_ops.py:13-92: `CustomOpLibrary(path)`,
 * destination-passing ops whose outputs come first). A kernel directory holds `.cu` files; every op
 * `NAME` of the directory is one function
 *
 *     extern "C" int32_t NAME(const b200_user_tensor* outputs, int32_t num_outputs,
 *                             const b200_user_tensor* inputs, int32_t num_inputs, void* stream);
 *
 * that enqueues its work on `stream` (a cudaStream_t) and returns 0, or a non-zero code that the
 * caller raises as an error. The output tensors are allocated by the caller (destination passing);
 * the function must not allocate device memory nor synchronise, so that it can be captured into a
 * CUDA graph like the library's own kernels. Tensors are described in elements, not bytes. */
#ifndef B200_USER_OP_H
#define B200_USER_OP_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_USER_MAX_RANK 8

typedef enum b200_user_dtype {
  B200_USER_U8 = 0,
  B200_USER_I8 = 1,
  B200_USER_I16 = 2,
  B200_USER_I32 = 3,
  B200_USER_I64 = 4,
  B200_USER_F16 = 5,
  B200_USER_BF16 = 6,
  B200_USER_F32 = 7,
  B200_USER_F64 = 8,
  B200_USER_BOOL = 9
} b200_user_dtype;

typedef struct b200_user_tensor {
  void* data;     /* device pointer of element [0, 0, ...] */
  int32_t dtype;  /* b200_user_dtype */
  int32_t rank;   /* 0 .. B200_USER_MAX_RANK */
  int64_t shape[B200_USER_MAX_RANK];
  int64_t strides[B200_USER_MAX_RANK]; /* in elements */
} b200_user_tensor;

typedef int32_t (*b200_user_op_fn)(const b200_user_tensor* outputs, int32_t num_outputs,
                                   const b200_user_tensor* inputs, int32_t num_inputs, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_USER_OP_H */
