/* C interface of libfdb200_runner.so: replays a plan file written by Runtime.export_plan (Python) in a process
 * that has no Python. Link with -lfdb200_runner; the kernel library libfdb200_kernels.so is opened by path.
 *
 *   void* plan = fdplan_load("model.fdplan", "/path/to/libfdb200_kernels.so");
 *   fdplan_set_input(plan, 0, pixels, fdplan_io_bytes(plan, 0, 0));   // dense, in the input's own dimension order
 *   fdplan_run(plan);                                                // one CUDA graph launch from the third call on
 *   fdplan_get_output(plan, 0, out, fdplan_io_bytes(plan, 1, 0));
 *   fdplan_destroy(plan);
 *
 * Every function that returns int gives 0 on success; fdplan_last_error() describes the last failure of the
 * calling thread. dtype codes: 0 fp16, 1 bf16, 2 fp32, 3 uint8, 4 int32, 5 int64, 6 fp8 e4m3, 7 int8, 8 bool. */
#ifndef FD_PLAN_RUNNER_H_
#define FD_PLAN_RUNNER_H_

#ifdef __cplusplus
extern "C" {
#endif

void* fdplan_load(const char* plan_path, const char* kernels_lib_path);
void fdplan_destroy(void* plan);
const char* fdplan_last_error(void);
int fdplan_num_ops(void* plan);
int fdplan_num_inputs(void* plan);
int fdplan_num_outputs(void* plan);
const char* fdplan_io_name(void* plan, int is_output, int index);
/* dims has room for 8 entries; returns the number of dimensions or -1 */
int fdplan_io_desc(void* plan, int is_output, int index, int* dtype, long long* dims);
unsigned long long fdplan_io_bytes(void* plan, int is_output, int index);
int fdplan_set_input(void* plan, int index, const void* host, unsigned long long bytes);
int fdplan_run(void* plan);
int fdplan_get_output(void* plan, int index, void* host, unsigned long long bytes);
/* milliseconds per run over `iters` graph launches, timed with CUDA events; -1 on error */
double fdplan_time(void* plan, int iters);

#ifdef __cplusplus
}
#endif
#endif
