// Flat C binding over the public C++ Tensor / nn interface (see
// include/mg_tensor_c.h).  Only public members are used, so this file builds
// unchanged against the reference's own sources (that build is the "true
// reference" checker library) and against the B200 backend.
#include "mg_tensor_c.h"

#include "micrograd/Tensor.h"
#include "micrograd/Utils.h"
#include "micrograd/nn.h"

#include <cstdlib>
#include <cstring>
#include <exception>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

struct mgt_tensor_s {
  std::shared_ptr<Tensor> p;
};
struct mgt_linear_s {
  Linear l;
  mgt_linear_s(size_t i, size_t o) : l(i, o) {}
};
struct mgt_sgd_s {
  SGD s;
  mgt_sgd_s(std::vector<std::shared_ptr<Tensor>> ps, double lr) : s(std::move(ps), lr) {}
};

namespace {

thread_local std::string g_err;

void record_current_exception() {
  try {
    throw;
  } catch (const std::invalid_argument &e) {
    g_err = std::string("invalid_argument: ") + e.what();
  } catch (const std::out_of_range &e) {
    g_err = std::string("out_of_range: ") + e.what();
  } catch (const std::runtime_error &e) {
    g_err = std::string("runtime_error: ") + e.what();
  } catch (const std::bad_alloc &e) {
    g_err = std::string("bad_alloc: ") + e.what();
  } catch (const std::exception &e) {
    g_err = std::string("exception: ") + e.what();
  } catch (...) {
    g_err = "unknown: non-standard exception";
  }
}

mgt_tensor wrap(std::shared_ptr<Tensor> p) {
  if (!p) {
    g_err = "runtime_error: null tensor";
    return nullptr;
  }
  return new mgt_tensor_s{std::move(p)};
}

template <class F> mgt_tensor guard_tensor(F &&f) {
  try {
    return wrap(f());
  } catch (...) {
    record_current_exception();
    return nullptr;
  }
}

template <class F> int guard_int(F &&f) {
  try {
    f();
    return 0;
  } catch (...) {
    record_current_exception();
    return -1;
  }
}

char *dup_string(const std::string &s) {
  char *out = static_cast<char *>(std::malloc(s.size() + 1));
  if (out) {
    std::memcpy(out, s.c_str(), s.size() + 1);
  }
  return out;
}

std::vector<size_t> index_vec(const size_t *idx, size_t n) {
  return std::vector<size_t>(idx, idx + n);
}

} // namespace

extern "C" {

const char *mgt_last_error(void) { return g_err.c_str(); }

mgt_tensor mgt_new(const size_t *shape, size_t ndim, const double *data, size_t ndata) {
  return guard_tensor([&] {
    std::vector<size_t> shp(shape, shape + ndim);
    if (data == nullptr) {
      return std::make_shared<Tensor>(shp);
    }
    return std::make_shared<Tensor>(shp, std::vector<double>(data, data + ndata));
  });
}

void mgt_release(mgt_tensor t) { delete t; }

size_t mgt_ndim(mgt_tensor t) { return t->p->shape().size(); }

void mgt_shape(mgt_tensor t, size_t *out) {
  const auto &s = t->p->shape();
  for (size_t i = 0; i < s.size(); i++) {
    out[i] = s[i];
  }
}

size_t mgt_size(mgt_tensor t) { return t->p->size(); }

// With the B200 backend the getters read through the const accessors: a mutable
// data()/grad() reference would mark the device copy stale and force a re-upload
// before the next kernel.  The reference has only the mutable accessors.
#ifdef MG_B200_EXTENSIONS
#define MGT_READ_VIEW(tensor) std::as_const(*(tensor))
#else
#define MGT_READ_VIEW(tensor) (*(tensor))
#endif

int mgt_get_data(mgt_tensor t, double *out, size_t n) {
  return guard_int([&] {
    auto &v = MGT_READ_VIEW(t->p).data();
    if (n != v.size()) {
      throw std::invalid_argument("mgt_get_data: size mismatch");
    }
    std::memcpy(out, v.data(), n * sizeof(double));
  });
}

int mgt_get_grad(mgt_tensor t, double *out, size_t n) {
  return guard_int([&] {
    auto &v = MGT_READ_VIEW(t->p).grad();
    if (n != v.size()) {
      throw std::invalid_argument("mgt_get_grad: size mismatch");
    }
    std::memcpy(out, v.data(), n * sizeof(double));
  });
}

int mgt_set_data(mgt_tensor t, const double *src, size_t n) {
  return guard_int([&] {
    auto &v = t->p->data();
    if (n != v.size()) {
      throw std::invalid_argument("mgt_set_data: size mismatch");
    }
    std::memcpy(v.data(), src, n * sizeof(double));
  });
}

int mgt_set_grad(mgt_tensor t, const double *src, size_t n) {
  return guard_int([&] {
    auto &v = t->p->grad();
    if (n != v.size()) {
      throw std::invalid_argument("mgt_set_grad: size mismatch");
    }
    std::memcpy(v.data(), src, n * sizeof(double));
  });
}

double mgt_at(mgt_tensor t, const size_t *idx, size_t nidx) {
  const Tensor &ct = *t->p;
  return ct.at(index_vec(idx, nidx));
}

double mgt_grad_at(mgt_tensor t, const size_t *idx, size_t nidx) {
  const Tensor &ct = *t->p;
  return ct.grad_at(index_vec(idx, nidx));
}

int mgt_set_at(mgt_tensor t, const size_t *idx, size_t nidx, double v) {
  return guard_int([&] { t->p->at(index_vec(idx, nidx)) = v; });
}

int mgt_to(mgt_tensor t, int backend) {
  return guard_int([&] { t->p->to(static_cast<micrograd::Backend>(backend)); });
}

int mgt_backend(mgt_tensor t) { return static_cast<int>(t->p->backend()); }

mgt_tensor mgt_binary(mgt_tensor a, mgt_tensor b, int op) {
  return guard_tensor([&]() -> std::shared_ptr<Tensor> {
    switch (op) {
    case MGT_ADD:
      return a->p->add(b->p);
    case MGT_SUB:
      return a->p->sub(b->p);
    case MGT_MUL:
      return a->p->mul(b->p);
    case MGT_DIV:
      return a->p->div(b->p);
    case MGT_MATMUL:
      return a->p->matmul(b->p);
    default:
      throw std::invalid_argument("mgt_binary: unknown op");
    }
  });
}

mgt_tensor mgt_scalar(mgt_tensor a, double s, int op) {
  return guard_tensor([&]() -> std::shared_ptr<Tensor> {
    switch (op) {
    case MGT_SADD:
      return a->p->add(s);
    case MGT_SSUB:
      return a->p->sub(s);
    case MGT_SMUL:
      return a->p->mul(s);
    case MGT_SDIV:
      return a->p->div(s);
    case MGT_POW:
      return a->p->pow(s);
    default:
      throw std::invalid_argument("mgt_scalar: unknown op");
    }
  });
}

mgt_tensor mgt_unary(mgt_tensor a, int op) {
  return guard_tensor([&]() -> std::shared_ptr<Tensor> {
    switch (op) {
    case MGT_RELU:
      return a->p->relu();
    case MGT_SIGMOID:
      return a->p->sigmoid();
    case MGT_TANH:
      return a->p->tanh();
    case MGT_SUM:
      return a->p->sum();
#ifdef MG_B200_EXTENSIONS
    case MGT_EXP:
      return a->p->exp();
#endif
    default:
      throw std::invalid_argument("mgt_unary: unknown op");
    }
  });
}

int mgt_backward(mgt_tensor t) {
  return guard_int([&] { t->p->backward(); });
}

int mgt_zero_grad(mgt_tensor t) {
  return guard_int([&] { t->p->zero_grad(); });
}

mgt_tensor mgt_mse_loss(mgt_tensor prediction, mgt_tensor target) {
  return guard_tensor([&] { return mse_loss(prediction->p, target->p); });
}

mgt_tensor mgt_avg_pool_2x2(mgt_tensor input) {
  return guard_tensor([&] { return avg_pool_2x2(input->p); });
}

mgt_linear mgt_linear_new(size_t in_features, size_t out_features) {
  try {
    return new mgt_linear_s(in_features, out_features);
  } catch (...) {
    record_current_exception();
    return nullptr;
  }
}

void mgt_linear_release(mgt_linear l) { delete l; }

mgt_tensor mgt_linear_forward(mgt_linear l, mgt_tensor input) {
  return guard_tensor([&] { return l->l.forward(input->p); });
}

mgt_tensor mgt_linear_weights(mgt_linear l) {
  return guard_tensor([&] { return l->l.weights(); });
}

mgt_tensor mgt_linear_bias(mgt_linear l) {
  return guard_tensor([&] { return l->l.bias(); });
}

mgt_sgd mgt_sgd_new(const mgt_tensor *params, size_t nparams, double lr) {
  try {
    std::vector<std::shared_ptr<Tensor>> ps;
    ps.reserve(nparams);
    for (size_t i = 0; i < nparams; i++) {
      ps.push_back(params[i]->p);
    }
    return new mgt_sgd_s(std::move(ps), lr);
  } catch (...) {
    record_current_exception();
    return nullptr;
  }
}

void mgt_sgd_release(mgt_sgd s) { delete s; }

int mgt_sgd_step(mgt_sgd s) {
  return guard_int([&] { s->s.step(); });
}

int mgt_sgd_zero_grad(mgt_sgd s) {
  return guard_int([&] { s->s.zero_grad(); });
}

int mgt_save_model(const char *path, mgt_linear l1, mgt_linear l2) {
  return guard_int([&] { save_model(path, l1->l, l2->l); });
}

int mgt_load_model(const char *path, mgt_linear l1, mgt_linear l2) {
  return guard_int([&] { load_model(path, l1->l, l2->l); });
}

char *mgt_to_dot(mgt_tensor t) {
  try {
    return dup_string(to_dot(t->p));
  } catch (...) {
    record_current_exception();
    return nullptr;
  }
}

char *mgt_format_scalar(const char *op, double scalar) {
  try {
    return dup_string(format_scalar(op, scalar));
  } catch (...) {
    record_current_exception();
    return nullptr;
  }
}

void mgt_free_str(char *s) { std::free(s); }

#ifdef MG_B200_EXTENSIONS

mgt_tensor mgt_sum_axis(mgt_tensor a, int axis) {
  return guard_tensor([&] { return a->p->sum(axis); });
}

mgt_tensor mgt_softmax_cross_entropy(mgt_tensor logits, mgt_tensor labels, double denom) {
  return guard_tensor([&] { return softmax_cross_entropy(logits->p, labels->p, denom); });
}

mgt_tensor mgt_softmax_cross_entropy_host(mgt_tensor logits, const int *labels_host, size_t nrows,
                                          double denom) {
  return guard_tensor([&] {
    return softmax_cross_entropy(logits->p, std::vector<int>(labels_host, labels_host + nrows),
                                 denom);
  });
}

mgt_tensor mgt_new_from_host(const size_t *shape, size_t ndim, const double *values) {
  return guard_tensor(
      [&] { return Tensor::from_host(std::vector<size_t>(shape, shape + ndim), values); });
}

int mgt_comm_rank(void) { return micrograd::comm_rank(); }
int mgt_comm_world(void) { return micrograd::comm_world(); }

int mgt_argmax_rows(mgt_tensor x, int *out, size_t nrows) {
  return guard_int([&] {
    std::vector<int> ids = argmax_rows(x->p);
    if (ids.size() != nrows) {
      throw std::invalid_argument("mgt_argmax_rows: size mismatch");
    }
    std::memcpy(out, ids.data(), nrows * sizeof(int));
  });
}

mgt_tensor mgt_linear_forward_relu(mgt_linear l, mgt_tensor input) {
  return guard_tensor([&] { return l->l.forward_relu(input->p); });
}

int mgt_set_requires_grad(mgt_tensor t, int flag) {
  return guard_int([&] { t->p->set_requires_grad(flag != 0); });
}

int mgt_sync(void) {
  return guard_int([&] { micrograd::synchronize(); });
}

int mgt_comm_unique_id(char *out128) {
  return guard_int([&] { micrograd::comm_unique_id(out128); });
}

int mgt_comm_init(const char *id128, int rank, int world) {
  return guard_int([&] { micrograd::comm_init(id128, rank, world); });
}

int mgt_comm_shutdown(void) {
  return guard_int([&] { micrograd::comm_shutdown(); });
}

int mgt_sgd_enable_allreduce(mgt_sgd s) {
  return guard_int([&] { s->s.enable_allreduce(); });
}

int mgt_copy_from_host(mgt_tensor t, const double *values, size_t n) {
  return guard_int([&] {
    if (n != t->p->size()) {
      throw std::invalid_argument("mgt_copy_from_host: size mismatch");
    }
    t->p->copy_from_host(values);
  });
}

int mgt_prefetch_from_host(mgt_tensor t, const double *values, size_t n) {
  return guard_int([&] {
    if (n != t->p->size()) {
      throw std::invalid_argument("mgt_prefetch_from_host: size mismatch");
    }
    t->p->prefetch_from_host(values);
  });
}

namespace {
// The one recorded step this flat binding offers; replaced by a fresh object when
// the caller abandons it.
std::unique_ptr<micrograd::RecordedStep> g_recorded_step = std::make_unique<micrograd::RecordedStep>();
}

int mgt_record_abandon(void) {
  return guard_int([&] { g_recorded_step = std::make_unique<micrograd::RecordedStep>(); });
}

int mgt_record_begin(void) {
  return guard_int([&] { g_recorded_step->begin(); });
}

int mgt_record_end(void) {
  return guard_int([&] { g_recorded_step->end(); });
}

int mgt_record_replay(void) {
  return guard_int([&] { g_recorded_step->replay(); });
}

int mgt_record_kernels(void) { return g_recorded_step->kernels(); }

#endif // MG_B200_EXTENSIONS

} // extern "C"
