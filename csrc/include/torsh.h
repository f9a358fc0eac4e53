/* C ABI of libtorsh_b200_host.so: tensors (fp32, host), elementwise / reduction / matmul / softmax / conv2d ops,
 * a linear layer, SGD and Adam optimizers, device queries and error reporting. Function names and calling
 * conventions follow the reference's C API (crates/torsh-ffi/src/c_api/{tensor,tensor_math,neural,optimizer,utils}.rs),
 * which is what its Node / Java / C# / Go / Swift / Ruby / R / Julia / Lua / MATLAB bindings are generated against.
 * All functions returning TorshStatus use 0 for success; torsh_get_last_error() describes the last failure of
 * the calling thread. Handles are opaque and must be released with the matching *_free. */
#ifndef TORSH_H
#define TORSH_H
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

#ifdef __cplusplus
}
#endif
#endif
