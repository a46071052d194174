/*
 * sptorch_b200_hal.h -- the C-ABI a dynamically loaded sptorch backend exports.
 *
 * These are the 20 entry points that sptorch's loader resolves by name
 * (crates/hal-ffi/src/lib.rs:176-214) and that its own contract header
 * declares (crates/hal-ffi/include/sptorch_hal.h:21-85).  The signatures
 * below are bit-for-bit the ones the loader binds, so libsptorch_b200.so can
 * be handed to FfiBackend::load() unchanged.  Everything behind them is
 * sm_100a CUDA; there is no CPU fallback: every call fails (non-zero /
 * NULL) when no B200-class device is usable.
 *
 * Conventions (same as the reference's):
 *   - int return: 0 = success, non-zero = failure.  No exception crosses the
 *     boundary.  A failed op never leaves `out` half written by a later op:
 *     errors are sticky and are reported again by sptorch_sync().
 *   - handles are opaque to the caller.  Here a handle IS the device address,
 *     so handles can be chained from op to op without touching the host.
 *   - sizes count f32 elements, never bytes.
 *   - ops are asynchronous on one library-owned stream; sptorch_copy_d2h
 *     returns only when the host buffer is valid; sptorch_sync drains all.
 *   - every function is thread-safe; init/shutdown are reference counted.
 */
#ifndef SPTORCH_B200_HAL_H
#define SPTORCH_B200_HAL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* lifecycle -- replaces sptorch_hal.h:24,27,30 (bound at hal-ffi/src/lib.rs:180-190) */
int         sptorch_backend_init(void);
void        sptorch_backend_shutdown(void);
const char* sptorch_backend_name(void);        /* "sptorch_b200"; valid until unload */

/* memory -- replaces sptorch_hal.h:35,38,41,44,47 (bound at hal-ffi/src/lib.rs:191-193,198-199) */
void* sptorch_alloc(size_t n);                 /* n f32 elements; NULL on failure; n==0 gives a valid 256-byte block */
void  sptorch_free(void* handle);              /* NULL tolerated */
int   sptorch_copy_h2d(const float* host, void* device, size_t n);
int   sptorch_copy_d2h(const void* device, float* host, size_t n);
int   sptorch_sync(void);

/* optional telemetry hook -- replaces sptorch_hal.h:59 (bound at hal-ffi/src/lib.rs:194-197).
 * queue_depth = operations enqueued on the stream and not yet known complete;
 * online = 1 while no sticky CUDA error has been recorded. */
int sptorch_query_runtime(uint32_t* queue_depth, uint32_t* online);

/* elementwise -- replaces sptorch_hal.h:63-70 (bound at hal-ffi/src/lib.rs:200-207) */
int sptorch_add_f32(const void* a, const void* b, void* out, size_t n);
int sptorch_mul_f32(const void* a, const void* b, void* out, size_t n);
int sptorch_neg_f32(const void* a, void* out, size_t n);
int sptorch_exp_f32(const void* a, void* out, size_t n);
int sptorch_log_f32(const void* a, void* out, size_t n);
int sptorch_relu_f32(const void* a, void* out, size_t n);
int sptorch_gelu_f32(const void* a, void* out, size_t n);   /* tanh form */
int sptorch_scale_f32(const void* a, float scalar, void* out, size_t n);

/* contractions -- replaces sptorch_hal.h:75,79 (bound at hal-ffi/src/lib.rs:208).
 * Row-major A[m,k] * B[k,n] -> C[m,n]; batched variant strides every
 * operand by its full matrix size. */
int sptorch_matmul_f32(const void* a, const void* b, void* out,
                       size_t m, size_t k, size_t n);
int sptorch_batch_matmul_f32(const void* a, const void* b, void* out,
                             size_t batch, size_t m, size_t k, size_t n);

/* row softmax over [rows, cols] -- replaces sptorch_hal.h:85 */
int sptorch_softmax_f32(const void* a, void* out, size_t rows, size_t cols);

#ifdef __cplusplus
}
#endif
#endif /* SPTORCH_B200_HAL_H */
