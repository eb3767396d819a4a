/* C ABI of libcarat_b200: the speculative-decoding step of the Carat Gemma-4 runtime, written for
 * NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every function returns 0 on success and a negative code on failure; the message is available
 *    from carat_b200_last_error() on the calling thread. Invalid arguments are rejected before any
 *    launch, so a failed call leaves device state untouched.
 *  - Pointers named device_* (and all tensor arguments) are device memory on the current device.
 *    `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *  - BF16 tensors are row-major unless stated; FP8 means e4m3 (finite, saturating, max 448).
 *  - Citations name the reference interface each entry point stands in for
 *    (paths inside the Gradiated/carat tree).
 */
#ifndef CARAT_B200_H
#define CARAT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Library ------------------------------------------------------------------------------------ */

/* Thread-local text of the most recent failure. */
const char *carat_b200_last_error(void);

/* ABI version of this header (bumped on incompatible changes). */
int carat_b200_abi_version(void);

/* Kernels that wait on hardware barriers give up after a bounded time and record a code in a
 * per-device word instead of hanging. Synchronises the device, returns the code in *code
 * (0 = healthy) and clears it. */
int carat_b200_device_error(int *code);

/* FP8 linear ---------------------------------------------------------------------------------- */

/* output[rows, output_width] = bf16((input_scale * weight_scale) *
 *                                   input_e4m3[rows, input_width] . weight_e4m3[output_width, input_width]^T)
 * with fp32 accumulation. rows <= 128, input_width a multiple of 16, operands 16-byte aligned.
 * `workspace` holds split-K partial sums and must be at least
 * carat_b200_fp8_linear_workspace_bytes() bytes (may be NULL when that is 0).
 * Replaces carat::Fp8Linear::run with Fp8Scaling::tensor (include/carat/linear.h:32-41,
 * cuda/linear.cu:645-803). */
int carat_b200_fp8_linear(const void *fp8_input, const float *device_input_scale,
                          const void *fp8_weight, const float *device_weight_scale,
                          void *bf16_output, int rows, int input_width, int output_width,
                          void *workspace, size_t workspace_bytes, void *stream);

size_t carat_b200_fp8_linear_workspace_bytes(int rows, int input_width, int output_width);

/* Fused LM head: device_tokens[row] = argmax_n bf16(scale * input[row] . weight[n]), ties to the
 * lowest n, without writing the logits. `device_keys` is rows * 8 bytes of scratch.
 * Replaces run_decode_lm_head + argmax_bf16_rows (cuda/batch_model_runner.cu:840-853,
 * cuda/ops.cu:935-981, 1566-1579). */
int carat_b200_fp8_linear_argmax(const void *fp8_input, const float *device_input_scale,
                                 const void *fp8_weight, const float *device_weight_scale,
                                 int *device_tokens, void *device_keys, int rows, int input_width,
                                 int output_width, void *stream);

/* Same contract as carat_b200_fp8_linear computed one output per thread without tensor cores.
 * A device-side cross-check for tests at sizes a CPU cannot finish; no step path calls it. */
int carat_b200_fp8_linear_check(const void *fp8_input, const float *device_input_scale,
                                const void *fp8_weight, const float *device_weight_scale,
                                void *bf16_output, int rows, int input_width, int output_width,
                                void *stream);

#ifdef __cplusplus
}
#endif

#endif /* CARAT_B200_H */
