/* libTHC for NVIDIA B200 (sm_100a): the C ABI of the gputorch / gpunn hot path.
 *
 * Drop-in boundary: the same C entry points, struct layouts and type semantics that the
 * reference's `libTHC.so` exports to its Lua bindings (gputorch/lib/THC/THC.h:4-11), restricted
 * to the conv / pool / threshold / GEMM / elementwise / reduction path, plus the plain-C cores of
 * the `gpunn_*` operators, which in the reference exist only behind `lua_State*` wrappers.
 * Everything is `extern "C"` with plain pointers, longs and floats.
 *
 * Differences a maintainer must know (all deliberate):
 *  - `THGPUStorage.data` is a CUDA DEVICE pointer (the reference kept a host-side view there and
 *    hid the device handle in `allocatorContext`, gputorch/lib/THC/THCStorage.cpp:44-50).
 *  - All work is asynchronous on one CUDA stream per host thread's current device; calls that
 *    return a host scalar or copy to host memory synchronise that stream.
 *  - Errors never exit the process (the reference did, gputorch/lib/THC/copyHelpers.cpp:27-32):
 *    a failing call records a thread-local message, invokes the installed handler if any, and
 *    returns leaving its outputs unspecified.  Poll `THGPUGetLastError()`.
 *  - There is no CPU fallback: without a CUDA device every compute entry point fails. */
#ifndef THC_B200_INC
#define THC_B200_INC

#include <stddef.h>

#ifdef __cplusplus
#define THC_API extern "C"
#else
#define THC_API extern
#endif

/* ---- TH host types this ABI exchanges with callers -------------------------------------------
 * Layout-identical to mcw_torch7_core/lib/TH/generic/THStorage.h:22-30 and
 * generic/THTensor.h (size, stride, nDimension, storage, storageOffset, refcount, flag).  When the
 * real TH.h has been included first, its definitions are used instead. */
#ifndef TH_INC
typedef struct THAllocator THAllocator;
#define THC_DECLARE_HOST_TYPES(NAME, T)                                                             \
  typedef struct TH##NAME##Storage {                                                                \
    T *data; long size; int refcount; char flag; THAllocator *allocator; void *allocatorContext;   \
  } TH##NAME##Storage;                                                                              \
  typedef struct TH##NAME##Tensor {                                                                 \
    long *size; long *stride; int nDimension; TH##NAME##Storage *storage; long storageOffset;      \
    int refcount; char flag;                                                                        \
  } TH##NAME##Tensor;
THC_DECLARE_HOST_TYPES(Byte, unsigned char)
THC_DECLARE_HOST_TYPES(Char, char)
THC_DECLARE_HOST_TYPES(Short, short)
THC_DECLARE_HOST_TYPES(Int, int)
THC_DECLARE_HOST_TYPES(Long, long)
THC_DECLARE_HOST_TYPES(Float, float)
THC_DECLARE_HOST_TYPES(Double, double)
#define TH_STORAGE_REFCOUNTED 1
#define TH_STORAGE_RESIZABLE 2
#define TH_STORAGE_FREEMEM 4
#define TH_TENSOR_REFCOUNTED 1
#endif

/* ---- torch.GPUStorage / torch.GPUTensor (gputorch/FFI.lua:5-29, gputorch/lib/THC/THCTensor.h:18-28) */
typedef struct THGPUStorage {
  float *data;            /* device pointer */
  long size;
  int refcount;
  char flag;
  THAllocator *allocator; /* unused, kept for layout */
  void *allocatorContext; /* (void*)(intptr_t)(device index + 1) of the owning device */
} THGPUStorage;

typedef struct THGPUTensor {
  long *size;
  long *stride;
  int nDimension;
  THGPUStorage *storage;
  long storageOffset;
  int refcount;
  char flag;
} THGPUTensor;

/* ---- library state, devices, errors (gputorch/lib/THC/THCGeneral.h:24-31, gputorch/init.cpp:10-66;
 * the reference's device functions are empty stubs, these are real) */
THC_API void THGPUInit(void);
THC_API void THGPUShutdown(void);
THC_API int THGPUGetDeviceCount(void);
THC_API void THGPUSetDevice(int device);          /* 0-based */
THC_API int THGPUGetDevice(void);
THC_API void THGPUSynchronize(void);               /* waits for the current device's stream */
THC_API void *THGPUGetStream(void);                /* cudaStream_t the library launches on */
THC_API void THGPUSetStream(void *cuda_stream);    /* adopt a caller-owned stream (NULL: library's own) */
THC_API const char *THGPUGetLastError(void);       /* NULL when the last calls on this thread succeeded */
THC_API void THGPUClearError(void);
THC_API void THGPUSetErrorHandler(void (*handler)(const char *msg, void *data), void *data);
/* Arithmetic of GEMM-shaped work: 0 = "fp32x3" (default; tcgen05 TF32 tensor cores with a 3-way
 * hi/lo operand split, FP32-accurate), 1 = "simt" (FP32 FMA on CUDA cores), 2 = "bf16" (opt-in,
 * single BF16 tensor-core product with FP32 accumulation; not FP32-accurate). */
THC_API void THGPUBlas_setMathMode(int mode);
THC_API int THGPUBlas_getMathMode(void);
/* Stall reporting of the tensor-core kernels (no counterpart in the reference, whose kernels have no waits).
 * Every mbarrier wait inside them is bounded: a wait that runs out makes its kernel, and every tensor-core
 * kernel queued behind it on the stream, leave without writing results, and the next call that synchronises
 * with the host (THGPUSynchronize, any copy to the host, get1d/2d, sumall/maxall/dot ..., the criterion's
 * loss) fails with an error instead of returning stale data.  `THGPUSetWaitLimit`: SM cycles one wait may
 * take (default 2^27, about 70 ms).  `THGPUStallProbe(limit)`: launches one warp that waits `limit` cycles on
 * a barrier nobody arrives on and then reports a stall exactly as an engine would (limit < 0: only marks the
 * host-side flag); it exists so that the reporting path can be tested without stalling a real kernel. */
THC_API void THGPUSetWaitLimit(long cycles);
THC_API long THGPUGetWaitLimit(void);
THC_API int THGPUStallProbe(long limit_cycles);
/* Count of kernels this library has launched on the calling thread since start. */
THC_API long THGPUKernelLaunchCount(void);
/* Count of stream-ordered device allocations the library has requested from the driver on the calling thread
 * (storages, and growth of the workspace arena that holds the temporaries of the entry points). */
THC_API long THGPUDeviceAllocCount(void);

/* ---- THGPUStorage (gputorch/lib/THC/THCStorage.cpp:7-198, THCStorageCopy.cpp:5-75) */
THC_API float *THGPUStorage_data(const THGPUStorage *self);
THC_API long THGPUStorage_size(const THGPUStorage *self);
THC_API void THGPUStorage_set(THGPUStorage *self, long index, float value);
THC_API float THGPUStorage_get(const THGPUStorage *self, long index);
THC_API THGPUStorage *THGPUStorage_new(void);
THC_API THGPUStorage *THGPUStorage_newWithSize(long size);
THC_API THGPUStorage *THGPUStorage_newWithData(float *device_data, long size); /* borrows; never frees */
THC_API void THGPUStorage_retain(THGPUStorage *self);
THC_API void THGPUStorage_free(THGPUStorage *self);
THC_API void THGPUStorage_fill(THGPUStorage *self, float value);
THC_API void THGPUStorage_resize(THGPUStorage *self, long size); /* keeps refcount (reference bug :196 not kept) */
THC_API void THGPUStorage_rawCopy(THGPUStorage *self, float *host_src);
THC_API void THGPUStorage_copy(THGPUStorage *self, THGPUStorage *src);
THC_API void THGPUStorage_copyGPU(THGPUStorage *self, THGPUStorage *src);
/* Copies from / to the seven host storage types (gputorch/lib/THC/THCStorageCopy.h:10-27; the reference stages
 * every non-Float type through a temporary FloatStorage on the host, THCStorageCopy.cpp:12-53).  Here the data
 * crosses the bus in its own type and a device kernel converts it with the C casts TH uses: (float)x to the
 * device, (type)x (truncation toward zero; narrow integers take the low bits of the int) back to the host. */
THC_API void THGPUStorage_copyByte(THGPUStorage *self, THByteStorage *src);
THC_API void THGPUStorage_copyChar(THGPUStorage *self, THCharStorage *src);
THC_API void THGPUStorage_copyShort(THGPUStorage *self, THShortStorage *src);
THC_API void THGPUStorage_copyInt(THGPUStorage *self, THIntStorage *src);
THC_API void THGPUStorage_copyLong(THGPUStorage *self, THLongStorage *src);
THC_API void THGPUStorage_copyFloat(THGPUStorage *self, THFloatStorage *src);
THC_API void THGPUStorage_copyDouble(THGPUStorage *self, THDoubleStorage *src);
THC_API void THByteStorage_copyGPU(THByteStorage *self, THGPUStorage *src);
THC_API void THCharStorage_copyGPU(THCharStorage *self, THGPUStorage *src);
THC_API void THShortStorage_copyGPU(THShortStorage *self, THGPUStorage *src);
THC_API void THIntStorage_copyGPU(THIntStorage *self, THGPUStorage *src);
THC_API void THLongStorage_copyGPU(THLongStorage *self, THGPUStorage *src);
THC_API void THFloatStorage_copyGPU(THFloatStorage *self, THGPUStorage *src);
THC_API void THDoubleStorage_copyGPU(THDoubleStorage *self, THGPUStorage *src);

/* ---- THGPUTensor object model (gputorch/lib/THC/THCTensor.cpp; host-side metadata only) */
THC_API THGPUStorage *THGPUTensor_storage(const THGPUTensor *self);
THC_API long THGPUTensor_storageOffset(const THGPUTensor *self);
THC_API int THGPUTensor_nDimension(const THGPUTensor *self);
THC_API long THGPUTensor_size(const THGPUTensor *self, int dim);
THC_API long THGPUTensor_stride(const THGPUTensor *self, int dim);
THC_API float *THGPUTensor_data(const THGPUTensor *self);
THC_API THGPUTensor *THGPUTensor_new(void);
THC_API THGPUTensor *THGPUTensor_newWithTensor(THGPUTensor *tensor);
THC_API THGPUTensor *THGPUTensor_newWithStorage(THGPUStorage *storage, long storageOffset, THLongStorage *size, THLongStorage *stride);
THC_API THGPUTensor *THGPUTensor_newWithStorage1d(THGPUStorage *storage, long storageOffset, long size0, long stride0);
THC_API THGPUTensor *THGPUTensor_newWithStorage2d(THGPUStorage *storage, long storageOffset, long size0, long stride0, long size1, long stride1);
THC_API THGPUTensor *THGPUTensor_newWithSize(THLongStorage *size, THLongStorage *stride);
THC_API THGPUTensor *THGPUTensor_newWithSize1d(long size0);
THC_API THGPUTensor *THGPUTensor_newWithSize2d(long size0, long size1);
THC_API THGPUTensor *THGPUTensor_newWithSize3d(long size0, long size1, long size2);
THC_API THGPUTensor *THGPUTensor_newWithSize4d(long size0, long size1, long size2, long size3);
THC_API THGPUTensor *THGPUTensor_newClone(THGPUTensor *self);
THC_API THGPUTensor *THGPUTensor_newContiguous(THGPUTensor *tensor);
THC_API THGPUTensor *THGPUTensor_newSelect(THGPUTensor *tensor, int dimension, long sliceIndex);
THC_API THGPUTensor *THGPUTensor_newNarrow(THGPUTensor *tensor, int dimension, long firstIndex, long size);
THC_API THGPUTensor *THGPUTensor_newTranspose(THGPUTensor *tensor, int dimension1, int dimension2);
THC_API void THGPUTensor_resize(THGPUTensor *tensor, THLongStorage *size, THLongStorage *stride);
THC_API void THGPUTensor_resizeAs(THGPUTensor *tensor, THGPUTensor *src);
THC_API void THGPUTensor_resize1d(THGPUTensor *tensor, long size0);
THC_API void THGPUTensor_resize2d(THGPUTensor *tensor, long size0, long size1);
THC_API void THGPUTensor_resize3d(THGPUTensor *tensor, long size0, long size1, long size2);
THC_API void THGPUTensor_resize4d(THGPUTensor *tensor, long size0, long size1, long size2, long size3);
THC_API void THGPUTensor_resize5d(THGPUTensor *tensor, long size0, long size1, long size2, long size3, long size4);
THC_API void THGPUTensor_set(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_setStorage(THGPUTensor *self, THGPUStorage *storage, long storageOffset, THLongStorage *size, THLongStorage *stride);
THC_API void THGPUTensor_narrow(THGPUTensor *self, THGPUTensor *src, int dimension, long firstIndex, long size);
THC_API void THGPUTensor_select(THGPUTensor *self, THGPUTensor *src, int dimension, long sliceIndex);
THC_API void THGPUTensor_transpose(THGPUTensor *self, THGPUTensor *src, int dimension1, int dimension2);
THC_API void THGPUTensor_squeeze(THGPUTensor *self, THGPUTensor *src);
THC_API int THGPUTensor_isContiguous(const THGPUTensor *self);
THC_API int THGPUTensor_isSameSizeAs(const THGPUTensor *self, const THGPUTensor *src);
THC_API long THGPUTensor_nElement(const THGPUTensor *self);
THC_API void THGPUTensor_retain(THGPUTensor *self);
THC_API void THGPUTensor_free(THGPUTensor *self);
THC_API void THGPUTensor_freeCopyTo(THGPUTensor *self, THGPUTensor *dst);
THC_API void THGPUTensor_set1d(THGPUTensor *tensor, long x0, float value);
THC_API void THGPUTensor_set2d(THGPUTensor *tensor, long x0, long x1, float value);
THC_API float THGPUTensor_get1d(const THGPUTensor *tensor, long x0);
THC_API float THGPUTensor_get2d(const THGPUTensor *tensor, long x0, long x1);

/* ---- copies (gputorch/lib/THC/THCTensorCopy.cpp:20-104 host<->device, :170-290 strided device copy) */
THC_API void THGPUTensor_copy(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_copyGPU(THGPUTensor *self, THGPUTensor *src);
/* host tensor of any of the seven TH types <-> device tensor (gputorch/lib/THC/THCTensorCopy.h:8-22); sizes may
 * differ as long as the element counts agree, strides on either side are honoured. */
THC_API void THGPUTensor_copyByte(THGPUTensor *self, THByteTensor *src);
THC_API void THGPUTensor_copyChar(THGPUTensor *self, THCharTensor *src);
THC_API void THGPUTensor_copyShort(THGPUTensor *self, THShortTensor *src);
THC_API void THGPUTensor_copyInt(THGPUTensor *self, THIntTensor *src);
THC_API void THGPUTensor_copyLong(THGPUTensor *self, THLongTensor *src);
THC_API void THGPUTensor_copyFloat(THGPUTensor *self, THFloatTensor *src);
THC_API void THGPUTensor_copyDouble(THGPUTensor *self, THDoubleTensor *src);
THC_API void THByteTensor_copyGPU(THByteTensor *self, THGPUTensor *src);
THC_API void THCharTensor_copyGPU(THCharTensor *self, THGPUTensor *src);
THC_API void THShortTensor_copyGPU(THShortTensor *self, THGPUTensor *src);
THC_API void THIntTensor_copyGPU(THIntTensor *self, THGPUTensor *src);
THC_API void THLongTensor_copyGPU(THLongTensor *self, THGPUTensor *src);
THC_API void THFloatTensor_copyGPU(THFloatTensor *self, THGPUTensor *src);
THC_API void THDoubleTensor_copyGPU(THDoubleTensor *self, THGPUTensor *src);

/* ---- serialisation (gputorch/torch/generic/Tensor.c:1150-1199 tensor write / read; generic/Storage.c:180-200
 * with the raw IO of gputorch/Storage.cpp:15-31; used by torch.save / torch.load and by nn.Module:clone(),
 * mcw_nn/Module.lua:104-114).  Records are the bytes the reference writes into a binary-mode THFile:
 *   storage:        long size; float data[size]
 *   tensor header:  int nDimension; long size[nd]; long stride[nd]; long storageOffset + 1
 * A Lua binding writes the header, then hands the storage to file:writeObject (which ends in
 * THGPUStorage_write), as the reference does.  THGPUTensor_write / _read are the whole record for hosts
 * without Lua: header, a long flag (1: a storage record follows; 0: none), the storage.  Storages shared by
 * several tensors are written once per tensor at this level (Lua's writeObject deduplicates by object index).
 * The file is a pair of callbacks that move exactly `nbytes` bytes and return the count moved; device data
 * is staged through the host in chunks of at most 16 MiB.  Each function returns 0, or 1 after recording an
 * error. */
typedef struct THGPUFile {
  long (*write)(void *ctx, const void *data, long nbytes);
  long (*read)(void *ctx, void *data, long nbytes);
  void *ctx;
} THGPUFile;
THC_API int THGPUStorage_write(const THGPUStorage *self, const THGPUFile *file);
THC_API int THGPUStorage_read(THGPUStorage *self, const THGPUFile *file);   /* resizes self to the recorded size */
THC_API int THGPUTensor_writeHeader(const THGPUTensor *self, const THGPUFile *file);
/* reads a header and points `self` at `storage` (already read; NULL only for an empty tensor) with that view */
THC_API int THGPUTensor_readHeader(THGPUTensor *self, THGPUStorage *storage, const THGPUFile *file);
THC_API int THGPUTensor_write(const THGPUTensor *self, const THGPUFile *file);
THC_API int THGPUTensor_read(THGPUTensor *self, const THGPUFile *file);     /* self gets a fresh storage */

/* ---- tensor math (gputorch/lib/THC/THCTensorMath.h:7-93; bodies THCTensorMath.cpp) */
THC_API void THGPUTensor_fill(THGPUTensor *self, float value);                                   /* :15-30 */
THC_API void THGPUTensor_zero(THGPUTensor *self);                                                /* :32-42 */
THC_API void THGPUTensor_zeros(THGPUTensor *r_, THLongStorage *size);                            /* :44-48 */
THC_API void THGPUTensor_ones(THGPUTensor *r_, THLongStorage *size);                             /* :50-54 */
THC_API void THGPUTensor_reshape(THGPUTensor *r_, THGPUTensor *t, THLongStorage *size);          /* :56-60 */
THC_API long THGPUTensor_numel(THGPUTensor *t);
THC_API void THGPUTensor_add(THGPUTensor *self, THGPUTensor *src, float value);                  /* :67-77 */
THC_API void THGPUTensor_mul(THGPUTensor *self, THGPUTensor *src, float value);                  /* :79-89 */
THC_API void THGPUTensor_div(THGPUTensor *self, THGPUTensor *src, float value);                  /* :91-101 */
THC_API void THGPUTensor_cadd(THGPUTensor *self, THGPUTensor *src1, float value, THGPUTensor *src2); /* :103-129 */
THC_API void THGPUTensor_cmul(THGPUTensor *self, THGPUTensor *src1, THGPUTensor *src2);          /* :131-146 */
THC_API void THGPUTensor_cdiv(THGPUTensor *self, THGPUTensor *src1, THGPUTensor *src2);          /* :148-163 */
THC_API float THGPUTensor_dot(THGPUTensor *self, THGPUTensor *src);                              /* :269-281 */
THC_API float THGPUTensor_minall(THGPUTensor *self);                                             /* :283-293 */
THC_API float THGPUTensor_maxall(THGPUTensor *self);                                             /* :295-305 */
THC_API float THGPUTensor_sumall(THGPUTensor *self);                                             /* :308-314 */
THC_API float THGPUTensor_meanall(THGPUTensor *self);
THC_API float THGPUTensor_prodall(THGPUTensor *self);                                            /* :316-322 */
/* No counterpart in the reference.  Sum of `n` contiguous floats at a DEVICE pointer into
 * device_result[0] (DEVICE pointer), asynchronously on `cuda_stream`, for callers that may not allocate
 * device memory (regions recorded for replay, fixed-budget serving loops, hosts that own all device
 * memory): it never calls cudaMalloc/cudaFree; its working memory is a fixed ~33 KB array inside the
 * library.  n in [1, 134217728]; larger inputs are refused.  The first call on a device resolves the
 * array's address and should precede any stream capture; calls that overlap on one GPU race on the
 * shared array.  Returns 0, or 1 after recording an error. */
THC_API int THGPUTensor_sumall_noalloc(const float *device_x, long n, float *device_result, void *cuda_stream);
/* Dim-wise reductions; `dim` is 0-based.  `indices` receives, as floats, the 1-based position of
 * the first extremum along `dim` (the convention of the reference's own GPU index kernel,
 * gputorch/lib/THC/gpunn-impl/Max.cpp:22-38; the reference's THGPUTensor_max never wrote it,
 * THCTensorMath.cpp:612-616).  `indices` may be NULL. */
THC_API void THGPUTensor_min(THGPUTensor *values, THGPUTensor *indices, THGPUTensor *src, long dim);
THC_API void THGPUTensor_max(THGPUTensor *values, THGPUTensor *indices, THGPUTensor *src, long dim);
THC_API void THGPUTensor_sum(THGPUTensor *self, THGPUTensor *src, long dim);                     /* :602-605 */
THC_API void THGPUTensor_mean(THGPUTensor *self, THGPUTensor *src, long dim);
THC_API void THGPUTensor_prod(THGPUTensor *self, THGPUTensor *src, long dim);                    /* :607-610 */
THC_API void THGPUTensor_addmv(THGPUTensor *self, float beta, THGPUTensor *t, float alpha, THGPUTensor *mat, THGPUTensor *vec); /* :624-695 */
THC_API void THGPUTensor_addmm(THGPUTensor *self, float beta, THGPUTensor *t, float alpha, THGPUTensor *mat1, THGPUTensor *mat2); /* :697-807 */
THC_API void THGPUTensor_addr(THGPUTensor *self, float beta, THGPUTensor *t, float alpha, THGPUTensor *vec1, THGPUTensor *vec2); /* :809-860 */

/* ---- pointwise math and whole-tensor norms (signatures gputorch/lib/THC/THCTensorMath.h:24-25,39-88; reference
 * bodies THCTensorMath.cpp:165-267, :862-1465).  Values follow the CPU TH functions
 * (mcw_torch7_core/lib/TH/generic/THTensorMath.c:274-290 clamp, :346-367 addcmul / addcdiv, :746-760 sign,
 * :1198-1234 comparisons, :1236-1300 unary functions, :1429-1521 normall / dist / varall / stdall): unary
 * functions within rel 1e-4 / abs 1e-5 of the C function of the element; comparisons write 1.0 / 0.0. */
THC_API void THGPUTensor_addcmul(THGPUTensor *self, THGPUTensor *t, float value, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_addcdiv(THGPUTensor *self, THGPUTensor *t, float value, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_log(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_log1p(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_exp(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_cos(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_acos(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_cosh(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_sin(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_asin(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_sinh(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_tan(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_atan(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_tanh(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_pow(THGPUTensor *self, THGPUTensor *src, float value);
THC_API void THGPUTensor_clamp(THGPUTensor *self, THGPUTensor *src, float min_value, float max_value);
THC_API void THGPUTensor_sqrt(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_ceil(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_floor(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_abs(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_sign(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_round(THGPUTensor *self, THGPUTensor *src);
THC_API void THGPUTensor_atan2(THGPUTensor *r_, THGPUTensor *tx, THGPUTensor *ty);
THC_API void THGPUTensor_ltValue(THGPUTensor *self_, THGPUTensor *src, float value);
THC_API void THGPUTensor_gtValue(THGPUTensor *self_, THGPUTensor *src, float value);
THC_API void THGPUTensor_leValue(THGPUTensor *self_, THGPUTensor *src, float value);
THC_API void THGPUTensor_geValue(THGPUTensor *self_, THGPUTensor *src, float value);
THC_API void THGPUTensor_eqValue(THGPUTensor *self_, THGPUTensor *src, float value);
THC_API void THGPUTensor_neValue(THGPUTensor *self_, THGPUTensor *src, float value);
THC_API void THGPUTensor_ltTensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_gtTensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_leTensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_geTensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_eqTensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2);
THC_API void THGPUTensor_neTensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2);
THC_API float THGPUTensor_varall(THGPUTensor *self);
THC_API float THGPUTensor_stdall(THGPUTensor *self);
THC_API float THGPUTensor_normall(THGPUTensor *self, float value);
THC_API float THGPUTensor_dist(THGPUTensor *self, THGPUTensor *src, float value);
/* p-norm along `dimension` (0-based), result of size 1 there (THTensorMath.c:1401-1427) */
THC_API void THGPUTensor_norm(THGPUTensor *self, THGPUTensor *src, float value, long dimension);

/* Every slice along `dimension` (0-based) whose p-norm exceeds maxnorm is scaled to maxnorm (THCTensorMath.cpp:1195-1222;
 * values as mcw_torch7_core/lib/TH/generic/THTensorMath.c:1447-1496). */
THC_API void THGPUTensor_renorm(THGPUTensor *self, THGPUTensor *src, float value, long dimension, float max_norm);
/* Index operations along `dim` (0-based) with a HOST vector of 1-based positions (THCTensorMath.cpp:1331-1465; values as
 * THTensorMath.c:69-172).  Positions outside the indexed dimension are refused before anything runs. */
THC_API void THGPUTensor_indexCopy(THGPUTensor *res_, int dim, THLongTensor *indices, THGPUTensor *src);
THC_API void THGPUTensor_indexFill(THGPUTensor *tensor, int dim, THLongTensor *index, float val);
THC_API void THGPUTensor_indexSelect(THGPUTensor *tensor, THGPUTensor *src, int dim, THLongTensor *index);

/* ---- BLAS on raw device pointers, column-major Fortran convention
 * (gputorch/lib/THC/THCBlas.cpp:249-288 gemm, :436-467 gemv, :470-483 axpy, :486-502 ger).
 * All leading dimensions are honoured; C is not read when beta == 0. */
THC_API void THGPUBlas_gemm(char transa, char transb, long m, long n, long k, float alpha,
                            const float *a, long lda, const float *b, long ldb, float beta,
                            float *c, long ldc);
THC_API void THGPUBlas_gemv(char trans, long m, long n, float alpha, const float *a, long lda,
                            const float *x, long incx, float beta, float *y, long incy);
THC_API void THGPUBlas_axpy(long n, float a, const float *x, long incx, float *y, long incy);
THC_API void THGPUBlas_ger(long m, long n, float alpha, const float *x, long incx,
                           const float *y, long incy, float *a, long lda);

/* ---- gpunn operator cores: what each `static int gpunn_<Op>_<method>(lua_State*)` of the
 * reference computes after it has pulled its arguments off the Lua stack.  A Lua wrapper reads
 * the same module-table fields and forwards them here.  Results are written in place into the
 * module's tensors, which these functions resize themselves, as in the reference.  Each returns
 * 0 on success and non-zero after recording an error.
 *
 * SpatialConvolutionMM: gputorch/lib/THC/gpunn-impl/SpatialConvolutionMM.cpp
 *   updateOutput :110-225, updateGradInput :227-311, accGradParameters :313-429.
 * `finput` (the reference's column buffer) receives, in the tensor-core math mode, the channels-last
 * copy of the input that updateOutput builds: a [1, N, H, W, C] tensor of the FP32 values when the layer
 * runs on the raw-operand engine (input and output planes multiples of 32), else the TF32 hi / lo
 * planes (a [2, N, H, W, C'] tensor, C' = C rounded up to 4); accGradParameters reads them back when their shape fits the input it is given, exactly as the CPU
 * nn path reuses the finput of its forward pass (mcw_nn/generic/SpatialConvolutionMM.c:284-346).
 * `fgradInput` (the reference's ones vector) is accepted for signature compatibility and left
 * untouched: the convolution is an implicit GEMM with no column matrix. */
THC_API int THGPUNN_SpatialConvolutionMM_updateOutput(THGPUTensor *input, THGPUTensor *output,
    THGPUTensor *weight, THGPUTensor *bias, THGPUTensor *finput, THGPUTensor *fgradInput,
    int kW, int kH, int dW, int dH, int padding);
THC_API int THGPUNN_SpatialConvolutionMM_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, THGPUTensor *weight, THGPUTensor *finput, THGPUTensor *fgradInput,
    int kW, int kH, int dW, int dH, int padding);
THC_API int THGPUNN_SpatialConvolutionMM_accGradParameters(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradWeight, THGPUTensor *gradBias, THGPUTensor *finput, THGPUTensor *fgradInput,
    int kW, int kH, int dW, int dH, int padding, float scale);
/* updateGradInput (skipped when gradInput is NULL) then accGradParameters in one call that transposes
 * gradOutput once; what an override of nn.Module:backward (mcw_nn/Module.lua, which calls the two
 * methods in turn) forwards to.  No counterpart function in the reference. */
THC_API int THGPUNN_SpatialConvolutionMM_backward(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, THGPUTensor *weight, THGPUTensor *gradWeight, THGPUTensor *gradBias,
    THGPUTensor *finput, THGPUTensor *fgradInput, int kW, int kH, int dW, int dH, int padding, float scale);
/* SpatialMaxPooling: gputorch/lib/THC/gpunn-impl/SpatialMaxPooling.cpp updateOutput :205-281,
 * updateGradInput :283-383 (which rejects dW != kW; this one follows the CPU nn semantics,
 * mcw_nn/generic/SpatialMaxPooling.c:147-254, and accepts overlapping windows). */
THC_API int THGPUNN_SpatialMaxPooling_updateOutput(THGPUTensor *input, THGPUTensor *output,
    THGPUTensor *indices, int kW, int kH, int dW, int dH);
THC_API int THGPUNN_SpatialMaxPooling_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, THGPUTensor *indices, int kW, int kH, int dW, int dH);
/* Threshold / ReLU: gputorch/lib/THC/gpunn-impl/Threshold.cpp :16-38, :53-81. */
THC_API int THGPUNN_Threshold_updateOutput(THGPUTensor *input, THGPUTensor *output, double threshold, double val);
THC_API int THGPUNN_Threshold_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, double threshold);
/* Classifier tail: gpunn-impl/LogSoftMax.cpp:116-194, gpunn-impl/ClassNLLCriterion.cpp:96-198
 * (targets are a float GPU tensor of 1-based class ids; loss averaged over the batch). */
THC_API int THGPUNN_LogSoftMax_updateOutput(THGPUTensor *input, THGPUTensor *output);
THC_API int THGPUNN_LogSoftMax_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, THGPUTensor *output);
THC_API int THGPUNN_ClassNLLCriterion_updateOutput(THGPUTensor *input, THGPUTensor *target,
    THGPUTensor *outputTensor, int sizeAverage);
THC_API int THGPUNN_ClassNLLCriterion_updateGradInput(THGPUTensor *input, THGPUTensor *target,
    THGPUTensor *gradInput, int sizeAverage);
/* SoftMax: gpunn-impl/SoftMax.cpp (CPU mcw_nn/generic/SoftMax.c:5-110; the exponential is the CPU's polynomial,
 * mcw_torch7_core/lib/TH/THLogAdd.c:56-86).  updateGradInput reads `output`, as the reference does. */
THC_API int THGPUNN_SoftMax_updateOutput(THGPUTensor *input, THGPUTensor *output);
THC_API int THGPUNN_SoftMax_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, THGPUTensor *output);
/* SpatialAveragePooling: gpunn-impl/SpatialAveragePooling.cpp updateOutput :66-126, updateGradInput :184-240.  As in
 * the reference (GPU and CPU, mcw_nn/generic/SpatialAveragePooling.c:66-75) the output is the window SUM.  Overlapping
 * windows are accepted in both directions (the reference GPU backward refuses dW != kW, :194-195). */
THC_API int THGPUNN_SpatialAveragePooling_updateOutput(THGPUTensor *input, THGPUTensor *output,
    int kW, int kH, int dW, int dH);
THC_API int THGPUNN_SpatialAveragePooling_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput,
    THGPUTensor *gradInput, int kW, int kH, int dW, int dH);
/* Parameter update over flat buffers.  momentum == 0: w -= lr*g, i.e. Module:updateParameters
 * (mcw_nn/Module.lua:75-82).  momentum != 0: v = momentum*v + g; w -= lr*v (not in the reference). */
THC_API int THGPUNN_SGD_update(THGPUTensor *weight, THGPUTensor *grad, THGPUTensor *velocity,
    float lr, float momentum);

/* ---- data-parallel gradient exchange (no counterpart in the reference, which has no multi-GPU code).
 * One communicator per rank (= process = GPU).  The flat gradient buffer is summed over the ranks bucket by
 * bucket on the communicator's own stream while the backward pass still runs on the library's stream, and each
 * bucket's SGD update runs right behind its all-reduce; no call synchronises with the host.  A watchdog thread
 * aborts the communicator when a queued bucket has not completed within the timeout (default 30 s) or the
 * transport reports an error: the next call then returns the error (THGPUComm_error) instead of blocking.
 *   id:     rank 0 calls THGPUComm_getUniqueId (128 bytes) and hands the bytes to the other ranks by any means.
 *   layout: THGPUComm_setBuckets(flat_grad, bounds, nbuckets): bucket b = elements [bounds[2b], bounds[2b+1]) in the
 *           order the backward pass finishes them; all ranks must pass equal numbers (checked across the ranks
 *           before any gradient traffic is queued).
 *   step:   THGPUComm_allReduceAsync(b) once per bucket as soon as its gradients are queued, THGPUComm_wait()
 *           before the next step touches parameters or gradients.
 * The transport is a table of callbacks; THGPUComm_new installs NCCL (libnccl.so.2, loaded at run time).  All
 * callbacks return 0 on success except `done` (1 completed, 0 pending, < 0 error) and `agree` (1 when every
 * rank passed the same values, 0 when not, < 0 error). */
typedef struct THGPUComm THGPUComm;
typedef struct THGPUCommBackend {
  int (*all_reduce)(void *ctx, int bucket, float *data, long begin, long count);  /* queue sum over ranks, in place */
  int (*set_update)(void *ctx, float *w, float *v, float lr, float momentum);     /* may be NULL */
  int (*done)(void *ctx, int bucket);
  int (*join)(void *ctx);                    /* order the caller's later work behind everything queued */
  int (*agree)(void *ctx, const long *values, int n);
  int (*abort)(void *ctx);
  void (*destroy)(void *ctx);
  void *ctx;
} THGPUCommBackend;
THC_API int THGPUComm_getUniqueId(void *id_out_128_bytes);
THC_API THGPUComm *THGPUComm_new(int world, int rank, const void *unique_id_128_bytes);
/* max_ctas > 0: at most that many thread blocks (SMs) per collective of this communicator; 0: NCCL's default. */
THC_API THGPUComm *THGPUComm_newWithOptions(int world, int rank, const void *unique_id_128_bytes, int max_ctas);
THC_API THGPUComm *THGPUComm_newWithBackend(int world, int rank, const THGPUCommBackend *backend);
THC_API void THGPUComm_free(THGPUComm *comm);
THC_API int THGPUComm_setTimeout(THGPUComm *comm, double seconds);
THC_API int THGPUComm_setBuckets(THGPUComm *comm, THGPUTensor *flat_grad, const long *bounds, int nbuckets);
/* v = momentum*v + g; w -= lr*v behind each bucket's all-reduce (flat_v NULL / momentum 0: w -= lr*g) */
THC_API int THGPUComm_setUpdate(THGPUComm *comm, THGPUTensor *flat_w, THGPUTensor *flat_v, float lr, float momentum);
THC_API int THGPUComm_allReduceAsync(THGPUComm *comm, int bucket);
THC_API int THGPUComm_wait(THGPUComm *comm);
THC_API const char *THGPUComm_error(THGPUComm *comm);   /* NULL while the communicator is healthy */

#endif
