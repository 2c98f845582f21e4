/*
 * mg_tensor_c.h — flat C binding over the C++ `Tensor` / `nn` API.
 *
 * The public C++ interface of micrograd (include/micrograd/Tensor.h:15-50 and
 * include/micrograd/nn.h:6-34 in the reference project) is a set of classes
 * handled through std::shared_ptr, which no FFI can bind directly.  This header
 * is the plain-C view of exactly that interface: one opaque handle per
 * shared_ptr<Tensor>, one function per public method.  Python (ctypes), Go (cgo)
 * or any other host can drive the autograd graph through it.
 *
 * The implementation (micrograd_b200/src/capi.cpp) uses only public members of
 * the C++ classes, so the same source file builds against any implementation of
 * those headers.  Entry points under MG_B200_EXTENSIONS bind the additive API
 * that only the B200 backend has.
 *
 * Error model: functions returning a handle return NULL on failure, functions
 * returning int return 0 on success and -1 on failure; mgt_last_error() then
 * gives "<exception class>: <what()>" for the calling thread, e.g.
 * "invalid_argument: Tensor shapes do not match".
 */
#ifndef MG_TENSOR_C_H
#define MG_TENSOR_C_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mgt_tensor_s *mgt_tensor; /* owns one std::shared_ptr<Tensor>   */
typedef struct mgt_linear_s *mgt_linear; /* owns one Linear                    */
typedef struct mgt_sgd_s *mgt_sgd;       /* owns one SGD                       */

const char *mgt_last_error(void);

/* ---- construction / destruction (Tensor.h:16-18) ---- */
/* data == NULL selects the zero-filling constructor Tensor(shape). */
mgt_tensor mgt_new(const size_t *shape, size_t ndim, const double *data, size_t ndata);
void mgt_release(mgt_tensor t);

/* ---- introspection (Tensor.h:41-50) ---- */
size_t mgt_ndim(mgt_tensor t);
void mgt_shape(mgt_tensor t, size_t *out);
size_t mgt_size(mgt_tensor t);
int mgt_get_data(mgt_tensor t, double *out, size_t n);      /* copies data()  */
int mgt_get_grad(mgt_tensor t, double *out, size_t n);      /* copies grad()  */
int mgt_set_data(mgt_tensor t, const double *src, size_t n); /* writes through data() */
int mgt_set_grad(mgt_tensor t, const double *src, size_t n); /* writes through grad() */
double mgt_at(mgt_tensor t, const size_t *idx, size_t nidx);
double mgt_grad_at(mgt_tensor t, const size_t *idx, size_t nidx);
int mgt_set_at(mgt_tensor t, const size_t *idx, size_t nidx, double v);
int mgt_to(mgt_tensor t, int backend); /* value of micrograd::Backend */
int mgt_backend(mgt_tensor t);

/* ---- ops (Tensor.h:20-36) ---- */
enum { MGT_ADD = 0, MGT_SUB = 1, MGT_MUL = 2, MGT_DIV = 3, MGT_MATMUL = 4 };
enum { MGT_SADD = 0, MGT_SSUB = 1, MGT_SMUL = 2, MGT_SDIV = 3, MGT_POW = 4 };
enum { MGT_RELU = 0, MGT_SIGMOID = 1, MGT_TANH = 2, MGT_SUM = 3,
       MGT_EXP = 4 /* extension */ };
mgt_tensor mgt_binary(mgt_tensor a, mgt_tensor b, int op);
mgt_tensor mgt_scalar(mgt_tensor a, double s, int op);
mgt_tensor mgt_unary(mgt_tensor a, int op);

/* ---- autograd (Tensor.h:38-39) ---- */
int mgt_backward(mgt_tensor t);
int mgt_zero_grad(mgt_tensor t);

/* ---- nn (nn.h) ---- */
mgt_tensor mgt_mse_loss(mgt_tensor prediction, mgt_tensor target);
mgt_tensor mgt_avg_pool_2x2(mgt_tensor input);
mgt_linear mgt_linear_new(size_t in_features, size_t out_features);
void mgt_linear_release(mgt_linear l);
mgt_tensor mgt_linear_forward(mgt_linear l, mgt_tensor input);
mgt_tensor mgt_linear_weights(mgt_linear l);
mgt_tensor mgt_linear_bias(mgt_linear l);
mgt_sgd mgt_sgd_new(const mgt_tensor *params, size_t nparams, double lr);
void mgt_sgd_release(mgt_sgd s);
int mgt_sgd_step(mgt_sgd s);
int mgt_sgd_zero_grad(mgt_sgd s);
int mgt_save_model(const char *path, mgt_linear l1, mgt_linear l2);
int mgt_load_model(const char *path, mgt_linear l1, mgt_linear l2);

/* ---- Utils.h ---- */
/* Returns a malloc()ed string; free it with mgt_free_str(). */
char *mgt_to_dot(mgt_tensor t);
char *mgt_format_scalar(const char *op, double scalar);
void mgt_free_str(char *s);

#ifdef MG_B200_EXTENSIONS
/* ---- additive API of the B200 backend (no counterpart in the reference) ---- */
mgt_tensor mgt_sum_axis(mgt_tensor a, int axis);
/* denom: divisor of the mean; 0 = number of rows. */
mgt_tensor mgt_softmax_cross_entropy(mgt_tensor logits, mgt_tensor labels, double denom);
/* labels_host: nrows class ids; uploads them inside the call. */
mgt_tensor mgt_softmax_cross_entropy_host(mgt_tensor logits, const int *labels_host, size_t nrows,
                                          double denom);
/* Tensor::from_host: uploads straight from caller memory (pinned or pageable). */
mgt_tensor mgt_new_from_host(const size_t *shape, size_t ndim, const double *values);
int mgt_comm_rank(void);
int mgt_comm_world(void);
int mgt_argmax_rows(mgt_tensor x, int *out, size_t nrows);
mgt_tensor mgt_linear_forward_relu(mgt_linear l, mgt_tensor input);
int mgt_set_requires_grad(mgt_tensor t, int flag);
int mgt_sync(void);
/* data-parallel training */
int mgt_comm_unique_id(char *out128);
int mgt_comm_init(const char *id128, int rank, int world);
int mgt_comm_shutdown(void);
int mgt_sgd_enable_allreduce(mgt_sgd s);
/* Tensor::copy_from_host and micrograd::RecordedStep (one recorded step per process here). */
int mgt_copy_from_host(mgt_tensor t, const double *values, size_t n);
int mgt_prefetch_from_host(mgt_tensor t, const double *values, size_t n); /* Tensor::prefetch_from_host */
int mgt_record_begin(void);
int mgt_record_end(void);
int mgt_record_replay(void);
int mgt_record_kernels(void);
int mgt_record_abandon(void); /* what ~RecordedStep does to a recording that was never ended */
#endif

#ifdef __cplusplus
}
#endif
#endif /* MG_TENSOR_C_H */
