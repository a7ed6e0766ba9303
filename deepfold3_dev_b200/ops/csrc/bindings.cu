// Operator registration: everything the Python side calls lives under torch.ops.df3.
#include <torch/library.h>
#include <torch/torch.h>

using torch::Tensor;

std::tuple<Tensor, Tensor, Tensor> df3_layer_norm_fwd(const Tensor&, const c10::optional<Tensor>&,
                                                      const c10::optional<Tensor>&, double);
std::tuple<Tensor, Tensor> df3_layer_norm_bwd(const Tensor&, const Tensor&, const c10::optional<Tensor>&,
                                              const Tensor&, const Tensor&, bool);
std::tuple<Tensor, Tensor, Tensor> df3_plane_layer_norm_fwd(const Tensor&, const c10::optional<Tensor>&,
                                                            const c10::optional<Tensor>&, double);
std::tuple<Tensor, Tensor> df3_plane_layer_norm_bwd(const Tensor&, const Tensor&, const c10::optional<Tensor>&, const Tensor&,
                                                    const Tensor&, bool);
int64_t df3_elementwise_status();
Tensor df3_swiglu_fwd(const Tensor&);
Tensor df3_swiglu_bwd(const Tensor&, const Tensor&);
Tensor df3_gated_bwd(const Tensor&, const Tensor&, const c10::optional<Tensor>&);
std::tuple<Tensor, Tensor> df3_sigmoid_gate_bwd(const Tensor&, const Tensor&, const Tensor&);
Tensor df3_dropout_shared(const c10::optional<Tensor>&, const Tensor&, int64_t, int64_t, int64_t, bool, double, int64_t,
                          const c10::optional<Tensor>&);
void df3_adamw_ema(Tensor, const Tensor&, Tensor, Tensor, const c10::optional<Tensor>&, const Tensor&, const Tensor&,
                   double, double, double, double, double, double, double, const c10::optional<Tensor>&);

void df3_register_ada_norm(torch::Library& m);

#ifdef DF3_WITH_GEMM
void df3_register_gemm(torch::Library& m);
const char* df3_gemm_features();
void df3_register_attention(torch::Library& m);
void df3_register_peer(torch::Library& m);
void df3_register_peer_exchange(torch::Library& m);
#endif

static std::string df3_features() {
  std::string f = "layer_norm,swiglu,dropout_add,adamw_ema,plane_layer_norm,ada_norm";
#ifdef DF3_WITH_GEMM
  f += ",";
  f += df3_gemm_features();
#endif
  return f;
}

TORCH_LIBRARY(df3, m) {
  m.def("features() -> str", &df3_features);
  m.def("elementwise_status() -> int", &df3_elementwise_status);
  m.def("bounds_checked() -> bool", []() {
#ifdef DF3_BOUNDS_CHECK
    return true;
#else
    return false;
#endif
  });
  m.def("layer_norm_fwd(Tensor x, Tensor? w, Tensor? b, float eps) -> (Tensor, Tensor, Tensor)", &df3_layer_norm_fwd);
  m.def("layer_norm_bwd(Tensor dy, Tensor x, Tensor? w, Tensor mean, Tensor rstd, bool want_wb) -> (Tensor, Tensor)",
        &df3_layer_norm_bwd);
  m.def("plane_layer_norm_fwd(Tensor x, Tensor? w, Tensor? b, float eps) -> (Tensor, Tensor, Tensor)", &df3_plane_layer_norm_fwd);
  m.def("plane_layer_norm_bwd(Tensor dy, Tensor x, Tensor? w, Tensor mean, Tensor rstd, bool want_wb) -> (Tensor, Tensor)",
        &df3_plane_layer_norm_bwd);
  m.def("swiglu_fwd(Tensor x) -> Tensor", &df3_swiglu_fwd);
  m.def("swiglu_bwd(Tensor dy, Tensor x) -> Tensor", &df3_swiglu_bwd);
  m.def("gated_bwd(Tensor dy, Tensor gp, Tensor? mask) -> Tensor", &df3_gated_bwd);
  m.def("sigmoid_gate_bwd(Tensor dy, Tensor g, Tensor other) -> (Tensor, Tensor)", &df3_sigmoid_gate_bwd);
  m.def("dropout_shared(Tensor? res, Tensor x, int A, int B, int C, bool share_rows, float p, int seed, Tensor? seed_dev=None) -> Tensor",
        &df3_dropout_shared);
  m.def("adamw_ema(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, Tensor? ema, Tensor decay, Tensor scale, "
        "float lr, float b1, float b2, float eps, float bc1, float bc2, float ema_w, Tensor(d!)? p16=None) -> ()",
        &df3_adamw_ema);
  df3_register_ada_norm(m);
#ifdef DF3_WITH_GEMM
  df3_register_gemm(m);
  df3_register_attention(m);
  df3_register_peer(m);
  df3_register_peer_exchange(m);
#endif
}
