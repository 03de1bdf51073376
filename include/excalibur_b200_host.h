/*
 * excalibur_b200 - C entry points of the C++ host layer (excalibur_b200/csrc/host/), for
 * harnesses that cannot include C++ headers (the Python tests and the benchmark).
 *
 * The host layer mirrors the reference's operation plug-in API and graph executor:
 *   glasssix::excalibur::operation<Dtype>, operation_reflector<Dtype>, REGISTE(...)
 *       (reference include/Excalibur/operation.hpp:109-374, operation_reflector.hpp:16-93)
 *   glasssix::excalibur::pipeline<Dtype>
 *       (reference include/Excalibur/pipeline.hpp:18-45)
 * C++ users include excalibur_b200/csrc/host/pipeline.hpp directly; these functions wrap
 * pipeline<float> and single operations created through the reflector.  LOG(FATAL) / CHECK
 * failures inside the host layer (which terminate the process in the reference,
 * include/Primitives/logger.hpp:101-118) are turned into the status EXB_HOST_FATAL here and the
 * message is kept for exb_host_last_error().
 */
#ifndef EXCALIBUR_B200_HOST_H_
#define EXCALIBUR_B200_HOST_H_

#include <stdint.h>

#include "excalibur_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define EXB_HOST_FATAL (-100)

EXB_API const char* exb_host_last_error(void);

/* 1 when an operation class is registered under `class_name` (e.g. "operation_convolution")
 * for pipeline<float>; mirrors operation_reflector<float>::create_object's key lookup. */
EXB_API int exb_host_registered(const char* class_name);

/* pipeline<float>(lines of a .phai file, .racy path or "" for seeded dummy weights, device)
 * - reference include/Excalibur/pipeline.hpp:26. */
EXB_API int exb_host_pipeline_create(const char* phai_text, const char* racy_path, int device,
                                     void** out);
EXB_API int exb_host_pipeline_destroy(void* p);
/* key: "fusion" (fused NHWC plan, default 1), "cuda_graph" (default 1), "profile" (0/1 =
 * disable_profiler / enable_profiler, reference pipeline.hpp:38-39), "h2d_chunks" (k sub-batches whose
 * copies overlap the previous sub-batch's kernels, default 1), "host_f16_threads" (t > 0: the input is
 * converted to fp16 by t host threads before the copy - half the PCIe bytes, identical results; default 0). */
EXB_API int exb_host_pipeline_set_option(void* p, const char* key, int value);
/* The host-side fp32 -> fp16 conversion "host_f16_threads" uses (round to nearest even; F16C where the CPU
 * has it, bit-level otherwise or when force_scalar != 0).  Needs no GPU. */
EXB_API int exb_host_convert_f32_to_f16(const float* src, uint16_t* dst, int64_t n, int threads, int force_scalar);
/* forward(): `input` is HOST memory, fp32 NCHW; it is wrapped, not copied (page-locked memory
 * makes the upload asynchronous).  The call returns when the outputs are back on the host. */
EXB_API int exb_host_pipeline_forward(void* p, const float* input, int N, int C, int H, int W);
EXB_API int exb_host_pipeline_num_outputs(void* p);
EXB_API int exb_host_pipeline_output_name(void* p, int i, char* buf, int cap);
/* Output or any feature map by name (pipeline::get_featmap, pipeline.hpp:32).  out == NULL
 * returns only the shape; the data is fp32 NCHW.  With the fused plan, "<name>:int8" returns the quantised form
 * that int8 convolutions read (raw integers -128..127 in fp32). */
EXB_API int exb_host_pipeline_get(void* p, const char* name, float* out, int64_t cap, int* shape4);
/* The host tensor an output of the last forward lives in (fp32 NCHW), without a copy: what
 * pipeline<float>::forward returns to a C++ caller.  Valid until the next forward. */
EXB_API int exb_host_pipeline_output_ptr(void* p, const char* name, const float** data, int* shape4);
/* Kernels launched by the last forward (-1 when run op by op) and their device time in ms. */
EXB_API int exb_host_pipeline_stats(void* p, int* launches, double* device_ms);
EXB_API int exb_host_pipeline_dump_profile(void* p, const char* path);
/* The writer behind dump_profile: n (name, begin, end) entries -> a chrome://tracing JSON file with one "B" / "E"
 * event pair per entry (reference: the profiler's dump, include/Primitives/profiler.hpp).  Needs no GPU. */
EXB_API int exb_host_write_chrome_trace(const char* path, int n, const char* const* names, const double* begin_ms,
                                        const double* end_ms);
/* Re-run the fused plan `iters` times on the input the last forward left on the device: no
 * host<->device copies, device time between CUDA events on the plan's stream in *ms. */
EXB_API int exb_host_pipeline_run_resident(void* p, int iters, double* ms);
/* Per-kernel device times of the last forward run with the profiler enabled. */
EXB_API int exb_host_pipeline_trace_size(void* p);
EXB_API int exb_host_pipeline_trace_entry(void* p, int i, char* name, int cap, double* begin_ms,
                                          double* end_ms);

/* One operation through the reflector, the way pipeline does it: create_object(param),
 * init_weights(FILE*) from `racy_path` (or init_weights() when NULL/""), forward_gpu on fp32
 * NCHW host arrays.  shapes = 4 ints per input.  out == NULL returns only the shape. */
EXB_API int exb_host_op_run(const char* type, const char* params, const char* racy_path, int device,
                            int n_in, const float* const* inputs, const int* shapes, float* out,
                            int64_t cap, int* out_shape4);

/* ---- pipeline<unsigned short>: the reference's fp16 Dtype (tensors of IEEE half bits,
 * src/Excalibur/operation.cpp:74-93,124-126).  `input` and the results are fp16 NCHW in HOST memory.  A network whose
 * fused plan can read fp16 planes (a 3-channel image in front of an fp16 stem convolution, W a multiple of 4) runs
 * that plan: the fp16 input crosses PCIe as it is - half the bytes of the fp32 form - and the results equal those of
 * pipeline<float> on the same values, rounded to fp16.  Other graphs run op by op.
 * Options: "fusion", "cuda_graph", "h2d_chunks" as for exb_host_pipeline_set_option. */
EXB_API int exb_host_pipeline_f16_create(const char* phai_text, const char* racy_path, int device, void** out);
EXB_API int exb_host_pipeline_f16_destroy(void* p);
EXB_API int exb_host_pipeline_f16_set_option(void* p, const char* key, int value);
EXB_API int exb_host_pipeline_f16_forward(void* p, const uint16_t* input, int N, int C, int H, int W);
/* Output or feature map by name as fp16; out == NULL returns only the shape. */
EXB_API int exb_host_pipeline_f16_get(void* p, const char* name, uint16_t* out, int64_t cap, int* shape4);
/* Kernels launched by the last forward (-1 when run op by op) and their device time in ms. */
EXB_API int exb_host_pipeline_f16_stats(void* p, int* launches, double* device_ms);

/* ---- one batch over several GPUs (glasssix::excalibur::sharded_pipeline, csrc/host/sharded.hpp) ----------
 * Images are independent: a batch of N images is cut into contiguous slices, slice r = [lo, hi) of
 * exb_host_shard_bounds(N, replicas, r), each run by its own pipeline<float> replica (one per entry of `devices`,
 * reference include/Excalibur/pipeline.hpp:24-26: a pipeline is bound to one device id) on its own host thread, and
 * every output is gathered by row offset.  No collective, no peer access. */
EXB_API int exb_host_shard_bounds(int total, int world, int rank, int* lo, int* hi);
/* parts[i]: part_rows[i] rows of row_elems floats; written one after the other into out.  Needs no GPU. */
EXB_API int exb_host_gather_rows(const float* const* parts, const int* part_rows, int n_parts, int64_t row_elems,
                                 float* out);
EXB_API int exb_host_sharded_create(const char* phai_text, const char* racy_path, const int* devices, int n_devices,
                                    void** out);
EXB_API int exb_host_sharded_destroy(void* p);
/* "fusion", "cuda_graph", "h2d_chunks": as exb_host_pipeline_set_option, applied to every replica. */
EXB_API int exb_host_sharded_set_option(void* p, const char* key, int value);
/* `input`: N images, fp32 NCHW, HOST memory (page-locked memory makes the uploads asynchronous). */
EXB_API int exb_host_sharded_forward(void* p, const float* input, int N, int C, int H, int W);
EXB_API int exb_host_sharded_num_outputs(void* p);
EXB_API int exb_host_sharded_output_name(void* p, int i, char* buf, int cap);
/* An output of the last forward, all N images; out == NULL returns only the shape. */
EXB_API int exb_host_sharded_get(void* p, const char* name, float* out, int64_t cap, int* shape4);
/* Device time of the slowest replica in the last forward, ms. */
EXB_API int exb_host_sharded_device_ms(void* p, double* ms);

#ifdef __cplusplus
}
#endif
#endif /* EXCALIBUR_B200_HOST_H_ */
