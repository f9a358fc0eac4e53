/* C ABI of libtorsh_b200_host.so: tensors (fp32, host), elementwise / reduction / matmul / softmax / conv2d ops,
 * a linear layer, SGD and Adam optimizers, device queries and error reporting. Function names and calling
 * conventions follow the reference's C API (crates/torsh-ffi/src/c_api/{tensor,tensor_math,neural,optimizer,utils}.rs),
 * which is what its Node / Java / C# / Go / Swift / Ruby / R / Julia / Lua / MATLAB bindings are generated against.
 * All functions returning TorshStatus use 0 for success; torsh_get_last_error() describes the last failure of
 * the calling thread. Handles are opaque and must be released with the matching *_free. */
#ifndef TORSH_H
#define TORSH_H
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int TorshStatus; /* 0 ok, 1 invalid argument, 2 shape mismatch, 3 out of memory, 4 not available */
typedef struct TorshTensor TorshTensor;
typedef struct TorshLinear TorshLinear;
typedef struct TorshOptimizer TorshOptimizer;

TorshStatus torsh_init(void);
void torsh_cleanup(void);
const char* torsh_version(void);
const char* torsh_get_last_error(void);
void torsh_set_random_seed(uint64_t seed);
void torsh_set_grad_enabled(int enabled);
int torsh_is_grad_enabled(void);
int torsh_cuda_is_available(void);
int torsh_cuda_device_count(void);
TorshStatus torsh_set_device(int index);

TorshTensor* torsh_tensor_new(const float* data, const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_from_data(const float* data, const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_zeros(const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_ones(const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_rand(const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_randn(const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_clone(const TorshTensor* t);
TorshTensor* torsh_tensor_detach(const TorshTensor* t);
void torsh_tensor_free(TorshTensor* t);
float* torsh_tensor_data(TorshTensor* t);
int torsh_tensor_ndim(const TorshTensor* t);
int64_t torsh_tensor_numel(const TorshTensor* t);
TorshStatus torsh_tensor_shape(const TorshTensor* t, int64_t* out, int capacity);
int torsh_tensor_dtype(const TorshTensor* t); /* always 0 = f32 */

TorshTensor* torsh_tensor_add(const TorshTensor* a, const TorshTensor* b);
TorshTensor* torsh_tensor_sub(const TorshTensor* a, const TorshTensor* b);
TorshTensor* torsh_tensor_mul(const TorshTensor* a, const TorshTensor* b);
TorshTensor* torsh_tensor_div(const TorshTensor* a, const TorshTensor* b);
TorshTensor* torsh_tensor_add_scalar(const TorshTensor* a, float s);
TorshTensor* torsh_tensor_mul_scalar(const TorshTensor* a, float s);
TorshTensor* torsh_tensor_matmul(const TorshTensor* a, const TorshTensor* b);
TorshTensor* torsh_tensor_reshape(const TorshTensor* a, const int64_t* shape, int ndim);
TorshTensor* torsh_tensor_transpose(const TorshTensor* a, int dim0, int dim1);
TorshTensor* torsh_tensor_relu(const TorshTensor* a);
TorshTensor* torsh_tensor_sigmoid(const TorshTensor* a);
TorshTensor* torsh_tensor_tanh(const TorshTensor* a);
TorshTensor* torsh_tensor_exp(const TorshTensor* a);
TorshTensor* torsh_tensor_log(const TorshTensor* a);
TorshTensor* torsh_tensor_sqrt(const TorshTensor* a);
TorshTensor* torsh_tensor_abs(const TorshTensor* a);
TorshTensor* torsh_tensor_sin(const TorshTensor* a);
TorshTensor* torsh_tensor_cos(const TorshTensor* a);
TorshTensor* torsh_tensor_sum_all(const TorshTensor* a);
TorshTensor* torsh_tensor_mean_all(const TorshTensor* a);
TorshTensor* torsh_tensor_max_all(const TorshTensor* a);
TorshTensor* torsh_tensor_min_all(const TorshTensor* a);
TorshTensor* torsh_tensor_sum_dim(const TorshTensor* a, int dim, int keepdim);
TorshTensor* torsh_tensor_mean_dim(const TorshTensor* a, int dim, int keepdim);
TorshTensor* torsh_tensor_softmax(const TorshTensor* a, int dim);
/* input [N,C,H,W], weight [O,C,kh,kw], optional bias [O] */
TorshTensor* torsh_tensor_conv2d(const TorshTensor* input, const TorshTensor* weight, const TorshTensor* bias, int stride,
                                 int padding);

TorshLinear* torsh_linear_new(int64_t in_features, int64_t out_features, int bias);
TorshTensor* torsh_linear_forward(TorshLinear* l, const TorshTensor* x);
/* Accumulates d(loss)/d(weight), d(loss)/d(bias) for the last forward input and returns d(loss)/d(input). */
TorshTensor* torsh_linear_backward(TorshLinear* l, const TorshTensor* grad_output);
TorshTensor* torsh_linear_weight(TorshLinear* l);
TorshTensor* torsh_linear_bias(TorshLinear* l);
void torsh_linear_free(TorshLinear* l);

TorshOptimizer* torsh_sgd_new(float lr, float momentum, float weight_decay, int nesterov);
TorshOptimizer* torsh_adam_new(float lr, float beta1, float beta2, float eps, float weight_decay, int decoupled);
TorshStatus torsh_optimizer_add_linear(TorshOptimizer* o, TorshLinear* l);
TorshStatus torsh_optimizer_step(TorshOptimizer* o);
TorshStatus torsh_optimizer_zero_grad(TorshOptimizer* o);
void torsh_optimizer_free(TorshOptimizer* o);


/* ---- remaining names of the reference's C surface ---- */
typedef TorshLinear TorshModule; /* the only module kind of the C surface */
void torsh_clear_last_error(void);
int torsh_has_error(void);
int torsh_get_device_type(void); /* 0 = host */
int torsh_get_device_id(void);
size_t torsh_cuda_device_memory(int device_id);
const char* torsh_cuda_device_name(int device_id);
size_t torsh_get_memory_usage(void);      /* bytes held by live tensors */
size_t torsh_get_peak_memory_usage(void);
TorshStatus torsh_reset_memory_tracking(void);
int torsh_get_num_threads(void);
TorshStatus torsh_set_num_threads(int n);
TorshStatus torsh_set_autocast(int enabled);
int torsh_is_autocast_enabled(void);
TorshStatus torsh_set_debug_mode(int enabled);
int torsh_is_debug_mode_enabled(void);
TorshStatus torsh_start_profiling(void);
const char* torsh_stop_profiling(void); /* JSON summary, valid until the next call */

size_t torsh_tensor_size(const TorshTensor* t);
TorshTensor* torsh_tensor_scalar(float value);
TorshTensor* torsh_tensor_eye(size_t n);
TorshTensor* torsh_tensor_linspace(double start, double end, size_t steps);
TorshTensor* torsh_tensor_sub_scalar(const TorshTensor* a, float s);
TorshTensor* torsh_tensor_div_scalar(const TorshTensor* a, float s);
TorshTensor* torsh_tensor_tan(const TorshTensor* a);
TorshStatus torsh_tensor_multiply(const TorshTensor* a, const TorshTensor* b, TorshTensor* result);
TorshTensor* torsh_tensor_max_dim(const TorshTensor* a, int dim);
TorshTensor* torsh_tensor_min_dim(const TorshTensor* a, int dim);
TorshStatus torsh_tensor_axpy_inplace(TorshTensor* target, const TorshTensor* source, float alpha);
TorshStatus torsh_tensor_adam_step_inplace(TorshTensor* param, const TorshTensor* grad, TorshTensor* m, TorshTensor* v, float lr,
                                           float beta1, float beta2, float eps, int64_t step);

TorshModule* torsh_linear_create(size_t in_features, size_t out_features, bool bias);
size_t torsh_linear_get_input_features(const TorshModule* m);
size_t torsh_linear_get_output_features(const TorshModule* m);
void torsh_module_free(TorshModule* m);
TorshOptimizer* torsh_sgd_create(float lr);
TorshOptimizer* torsh_adam_create(float lr, float beta1, float beta2, float eps);
TorshStatus torsh_sgd_step(TorshOptimizer* o);

#ifdef __cplusplus
}
#endif
#endif
