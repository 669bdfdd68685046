/*
 * nsl_shims.h -- entry points with NSL's own calling convention (i64 handles that are raw
 * pointers to NSL's #[repr(C)] structs), forwarding to the CUDA kernels of libnslq_b200.
 *
 * These are what the Rust runtime would call from the GPU arm of its existing functions; the
 * struct mirrors below are checked against NSL's field order with static_asserts in
 * nsl_b200/csrc/nsl_shims.cu.  Differences from the CPU originals, all forced by ownership
 * (docs/abi/README.md:100-113 of NSL: tensors are allocated and freed by the Rust allocator):
 * the result tensor is passed in by the caller (`out`), already allocated on the device with
 * shape [M,N] and dtype f32, instead of being returned; on success the functions return `out`.
 */
#ifndef NSL_SHIMS_H
#define NSL_SHIMS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* crates/nsl-runtime/src/tensor/mod.rs:202-224 */
typedef struct NslTensor {
    uint32_t magic;        /* 0x4E534C54 "NSLT" when live */
    void    *data;         /* device pointer when device > 0 */
    int64_t *shape;        /* host */
    int64_t *strides;      /* host */
    int64_t  ndim;
    int64_t  len;
    int64_t  refcount;
    uint8_t  device;       /* 0 = CPU, 1+ = CUDA device id (1-based) */
    uint16_t dtype;        /* 0 f64, 1 f32, 2 fp16, 3 bf16, 4 int8, 9 i32 */
    uint8_t  owns_data;
    int64_t  data_owner;
    uint8_t  slab_managed;
    int64_t  tape_id;
} NslTensor;

/* crates/nsl-runtime/src/quantize.rs:27-51 (buffers in host memory, as the reference allocates them) */
typedef struct NslQuantizedTensor {
    uint8_t *data;
    float   *scale;
    uint8_t *zero_point;
    int64_t *shape;
    int64_t  ndim;
    int64_t  dtype;        /* 0 = INT8, 1 = INT4 */
    int64_t  granularity;  /* 0 tensor, 1 channel, 2 group */
    int64_t  gran_axis;
    int64_t  group_size;
    int64_t  num_scales;
    int64_t  refcount;
} NslQuantizedTensor;

/* crates/nsl-runtime/src/awq.rs:29-45 (buffers in host memory) */
typedef struct NslAwqPackedWeight {
    uint8_t *data;
    double  *scales;
    double  *zeros;
    int64_t  k, n, group_size, num_groups;
    int64_t  refcount;
} NslAwqPackedWeight;

/*
 * GPU arm of nsl_awq_matmul (crates/nsl-runtime/src/awq.rs:261-310): input [M,K] on the device
 * (f32, fp16 or bf16), packed = NslAwqPackedWeight* (host buffers; uploaded and re-laid out once,
 * cached by pointer and device).  fp32 input reaches the 16-bit kernels split into three bf16 parts
 * whose sum is x exactly.  Null pointers: message on stderr and 0, like the original.
 */
int64_t nsl_awq_matmul_cuda(int64_t input, int64_t packed, int64_t group_size, int64_t out);
/* GPU arm of nsl_gptq_matmul (crates/nsl-runtime/src/gptq.rs:646-653): same computation. */
int64_t nsl_gptq_matmul_cuda(int64_t input, int64_t packed, int64_t group_size, int64_t bits, int64_t out);

/*
 * GPU arm of nsl_qtensor_matmul_mixed (crates/nsl-runtime/src/quantize.rs:547-585): x [...,K] on
 * the device @ dequantize(qw [K,N]); every dtype/granularity the original accepts.  INT4 weights
 * quantised per tensor, per channel along axis 1 or per group along axis 0 (group a multiple of 128,
 * K a multiple of 64) are re-laid out once and multiplied by the streaming / tensor-core W4A16
 * kernels; the other forms run a generic kernel.  Like the original it prints and aborts when qw is
 * not 2-D or the inner dimensions differ.
 */
int64_t nsl_qtensor_matmul_mixed_cuda(int64_t x, int64_t qw, int64_t out);

/*
 * GPU arms of the load-time quantisers for a weight that already lives on the device.  The host objects are
 * allocated by the caller exactly as the originals allocate them (host buffers; shape, dtype, granularity,
 * gran_axis, group_size, num_scales resp. k, n, group_size, num_groups filled in) and receive the
 * reference's bytes.  Each returns its output handle, or 0 after printing the reason.
 *   nsl_qtensor_quantize_cuda    nsl_qtensor_quantize   (crates/nsl-runtime/src/quantize.rs:283-426), f32 or f64 tensor
 *   nsl_qtensor_dequantize_cuda  nsl_qtensor_dequantize (quantize.rs:436-537) into a device tensor, f64 (what the
 *                                original returns) or f32
 *   nsl_awq_quantize_cuda        nsl_awq_quantize       (crates/nsl-runtime/src/awq.rs:233-260), weight [K,N]
 */
int64_t nsl_qtensor_quantize_cuda(int64_t tensor, int64_t qt);
int64_t nsl_qtensor_dequantize_cuda(int64_t qt, int64_t out);
int64_t nsl_awq_quantize_cuda(int64_t weight, int64_t group_size, int64_t packed_out);

/* Drops the device copies cached for a weight on every device (call from nsl_awq_free / nsl_qtensor_free). */
void nsl_quant_forget_cuda(int64_t weight);

/*
 * The CUDA stream (cudaStream_t as i64) on which the calling THREAD's shim calls launch; 0 = the
 * legacy default stream, which is also the initial setting.  NSL launches on a per-thread compute
 * stream (crates/nsl-runtime/src/cuda/mod.rs:1931-1940): the runtime passes that stream here once.
 */
void nsl_quant_set_stream_cuda(int64_t stream);

/*
 * Sizes the calling thread's device scratch (quantised activations of nsl_bitlinear_forward beyond
 * the built-in 512 KiB area, split rows of fp32 activations for the W4 kernels) on the current
 * device to at least `bytes`, so that later forward calls allocate nothing.  Without it the scratch
 * grows on first need (cudaMalloc inside that one call).  Returns `bytes`, or 0 on failure.
 */
int64_t nsl_quant_reserve_cuda(int64_t bytes);

/*
 * GPU arm of nsl_awq_pre_scale_weight (crates/nsl-runtime/src/awq.rs:330-383): out[r,c] =
 * weight[r,c] * scales[c]^alpha in f32.  weight and out: f32 [K,N] on the device; scales: HOST
 * pointer to scales_len floats, as in the original (0 or a length other than N = plain copy).  The
 * powers are taken on the host with the same libm powf, so the result is the original's bit for bit.
 */
int64_t nsl_awq_pre_scale_weight_cuda(int64_t weight, int64_t scales, int64_t scales_len, double alpha, int64_t out);

/*
 * BitLinear: NSL has no runtime entry point for it (crates/nsl-codegen/tests/bitnet_logit_match.rs:44-52),
 * so this trio is new.  pack: `packed_bytes` = LoadedTernaryWeight.packed_bytes in HOST memory
 * ([out_dim][hidden_dim/4], crates/nsl-codegen/src/bitnet/loader.rs:47-56), uploaded once; returns a
 * handle or 0 (0 also for bytes that hold the reserved code 0b11, which NSL's try_unpack_byte rejects:
 * crates/nsl-codegen/src/bitnet/pack.rs:60-67).  forward: x [M,hidden] on the device (f32/fp16/bf16),
 * out [M,out_dim] on the device (f32/fp16/bf16); returns out or 0.  Decode-sized calls use the
 * library's built-in scratch area; larger ones the thread's scratch (nsl_quant_reserve_cuda).
 */
int64_t nsl_bitlinear_pack(int64_t packed_bytes, int64_t out_dim, int64_t hidden_dim, double weight_scale);
int64_t nsl_bitlinear_forward(int64_t handle, int64_t x, int64_t out);
void    nsl_bitlinear_free(int64_t handle);

#ifdef __cplusplus
}
#endif
#endif /* NSL_SHIMS_H */
