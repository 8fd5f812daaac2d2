// The kernel libraries (one shared library per file of csrc/) and their C entry points.
//
// A library is opened when it is first needed, from the folder that holds this library
// (or $FRIDAY_BUILD_DIR).  If it is not there, the builder hook is asked for it (the
// Python package compiles the family with nvcc at that moment); without a hook, or if
// the library still cannot be opened, the call fails with a KernelError that says how to
// build.  Nothing falls back to another path.
#pragma once
#include <cuda_runtime.h>

#include <string>

#include "csrc/gemm_tc_fusion.h"

namespace friday {
namespace kernels {

typedef const char* (*last_error_fn)();

struct Rowwise {
    last_error_fn last_error;
    int (*embedding)(const int*, const void*, void*, int, int, int, int, cudaStream_t);
    int (*gather_rows)(const int*, const void*, void*, int, int, int, cudaStream_t);
    int (*rmsnorm)(const void*, const void*, int, void*, int, int, float, int, cudaStream_t);
    int (*swiglu)(const void*, void*, int, int, int, cudaStream_t);
    int (*gated_act)(const void*, void*, int, int, int, int, cudaStream_t);
    int (*rope_kv_write)(void*, const int*, const int*, const float*, int, int, int, int, void*, void*, const int*, int, int,
                         int, int, int, cudaStream_t);
    int (*advance)(int*, const int*, int*, int*, const int*, int*, int, cudaStream_t);
    int (*scale_rows)(void*, long long, float, int, cudaStream_t);
    int (*finish_logits)(float*, int, int, int, const void*, int, float, float, cudaStream_t);
    int (*random_normal)(void*, long long, int, unsigned long long, float, float, cudaStream_t);
};
struct GemmSimt {
    last_error_fn last_error;
    int (*gemm)(const void*, int, const void*, int, void*, int, const void*, int, const void*, int, int, int, int, int, int,
                cudaStream_t);
};
struct GemmTc {
    last_error_fn last_error;
    int (*fused)(const void*, const void*, void*, int, const void*, int, const void*, int, int, int, int, int, int, float*,
                 long long, int*, int, int*, int, int, int, int, int, const GemmFusion*, cudaStream_t);
    int (*plan)(int, int, int, int, int, int, int, long long*);
};
struct AttentionSimt {
    last_error_fn last_error;
    int (*run)(const void*, int, void*, const void*, const void*, const int*, int, int, const int*, const int*, int, int, int,
               int, int, float, int, float*, int, cudaStream_t);
    int (*masked)(const void*, int, void*, const void*, const void*, const int*, int, int, const int*, const int*, int, int, int,
                  int, int, int, int, float, float, int, float*, int, cudaStream_t);
};
struct AttentionWindow {
    last_error_fn last_error;
    int (*fits)(int, int, int);
    int (*run)(const void*, int, void*, const void*, const void*, const int*, int, int, const int*, const int*, const int*, int, int,
               int, int, int, int, int, int, float, float, cudaStream_t);
};
struct Residual {
    last_error_fn last_error;
    int (*norm_cast)(const void*, int, const void*, int, float, void*, int, int, int, float, cudaStream_t);
    int (*concat_cast)(const void*, const void*, int, void*, int, int, int, int, cudaStream_t);
    int (*add_scaled)(const float*, const void*, float, const void*, float, int, float*, long long, cudaStream_t);
    int (*kv_store)(const void*, int, int, int, int, int, int, const int*, const int*, void*, void*, const int*, int, int, int, int,
                    cudaStream_t);
    int (*token_input)(float*, const int*, const int*, const void*, int, int, int, const void*, const void*, const void*, int, int,
                       int, int, float, float*, int, cudaStream_t);
    int (*gelu_table)(const float*, const int*, const void*, int, int, int, void*, int, int, int, cudaStream_t);
    int (*rms_add)(float*, const float*, const void*, int, int, int, float, cudaStream_t);
    int (*layernorm_cast)(const void*, int, const void*, const void*, int, void*, int, int, int, float, cudaStream_t);
    int (*embed_rows)(const int*, const void*, int, float*, int, int, int, float, cudaStream_t);
    int (*embed_pos)(const int*, const int*, const void*, const void*, int, float*, int, int, int, int, cudaStream_t);
    int (*norm_shift)(const float*, const void*, int, const void*, int, void*, int, float*, long long, const int*, const int*, const int*,
                      const int*, int, int, int, float, int, cudaStream_t);
    int (*post_norm_add)(const float*, const float*, const void*, int, float, float, float*, const void*, int, float, void*, int, int, int,
                         cudaStream_t);
    int (*two_sided_act)(void*, long long, int, const void*, int, cudaStream_t);
    int (*embed_pair)(const int*, const int*, const int*, const int*, const int*, const int*, const void*, const void*, int, int*, float*, int,
                      int, int, int, long long, long long, cudaStream_t);
    int (*norm_conv)(const float*, const void*, const void*, int, const void*, int, int, void*, int, float*, long long, long long, const int*,
                     const int*, const int*, int, int, float, int, cudaStream_t);
    int (*norm_conv_state)(const float*, const void*, const void*, int, int, int, float*, long long, long long, const int*, const int*,
                           const int*, int, int, float, cudaStream_t);
    int (*rms_pair_add)(const float*, const float*, const float*, const void*, const void*, int, float, float, float*, int, int, cudaStream_t);
};
struct Recurrence {
    last_error_fn last_error;
    int (*shift_mix)(const void*, void*, const void* const*, int, int, const float*, long long, const int*, const int*, const int*,
                     int, int, int, cudaStream_t);
    int (*tanh_rows)(void*, long long, int, cudaStream_t);
    int (*scan)(const void*, int, const void*, int, const void*, int, const float*, const void*, int, const void*, int, float*,
                float*, long long, long long, const void*, int, const int*, const int*, const int*, const int*, int, int, int, int,
                int, int, float, float, int, float*, int, cudaStream_t);
    int (*scan_plan)(int, int, int, int, int, long long*);
    int (*head_norm_gate)(const float*, const void*, int, void*, const void*, int, int, const int*, int, int, int, float, float, int,
                          int, cudaStream_t);
};
struct Delta {
    last_error_fn last_error;
    int (*conv_prepare)(const void*, int, int, int, int, const void*, int, float*, const float*, long long, const int*, const int*,
                        const int*, int, int, int, int, int, float, float, int, int, cudaStream_t);
    int (*conv_state)(const void*, int, int, int, int, float*, long long, const int*, const int*, const int*, const int*, int, int, int,
                      int, int, int, cudaStream_t);
    int (*scan)(const float*, const void*, int, const void*, int, int, const void*, const void*, int, float*, float*, long long,
                long long, const int*, const int*, const int*, const int*, int, int, int, int, int, int, cudaStream_t);
    int (*general_prepare)(const void*, int, int, int, const float*, int, const float*, int, const void*, const void*, int, float*, int, int,
                           int, float, float, int, cudaStream_t);
    int (*general_scan)(const float*, const void*, int, int, float*, float*, long long, long long, const int*, const int*, const int*, int,
                        int, int, int, int, cudaStream_t);
};
struct AttentionPooled {
    last_error_fn last_error;
    int (*prepare)(void*, int, int, int, int, const void*, const void*, int, float, const float*, float, int, void*, void*, const int*, int,
                   int, const int*, const int*, int, int, int, int, int, int, int, cudaStream_t);
    int (*pool)(const void*, const void*, float*, float*, const int*, int, const int*, int, int, const int*, const int*, int, int, int, int,
                int, int, int, cudaStream_t);
    long long (*scratch_floats)(int, int, int, int);
    int (*rows)(const void*, int, int, void*, const void*, const void*, const float*, const float*, const int*, int, const int*, int, int,
                const int*, const int*, int, int, int, int, int, int, int, float, float, int, const void*, int, int, float*, int,
                cudaStream_t);
    int (*prompt_fits)(int, int, int);
    int (*prompt)(const void*, int, int, void*, const void*, const void*, const float*, const float*, const int*, int, const int*, int, int,
                  const int*, const int*, const int*, int, int, int, int, int, int, int, int, float, float, int, const void*, int,
                  cudaStream_t);
};
struct AttentionLatent {
    last_error_fn last_error;
    int (*rotate_pairs)(void*, int, const int*, const int*, const float*, float, int, int, int, int, int, int, cudaStream_t);
    int (*prepare)(const void*, int, int, int, void*, float*, const void*, int, float, const int*, const int*, const float*, float, int,
                   int, int, int, int, int, int, cudaStream_t);
    int (*head_linear)(const void*, int, int, int, int, const void*, int, int, void*, int, int, int, const void*, int, int, const int*,
                       int, int, int, int, cudaStream_t);
    int (*run)(const float*, float*, const void*, const void*, const int*, int, int, const int*, const int*, const void*, int, int,
               int, int, int, float, int, float*, int, cudaStream_t);
    int (*gather)(const void*, const void*, const int*, int, int, int, int, int, void*, void*, int, cudaStream_t);
    int (*softmax_split)(const float*, int, int, int, int, float, const void*, int, int, void*, void*, int, cudaStream_t);
    int (*key_concat)(const void*, const void*, int, int, int, int, void*, int, cudaStream_t);
    int (*gate_cast)(const float*, const void*, int, int, int, int, int, void*, int, cudaStream_t);
};
struct Routed {
    last_error_fn last_error;
    int (*route)(const float*, int, int, int, int, int, int*, float*, float*, cudaStream_t);
    int (*scale_by_route)(void*, const float*, int, int, int, int, cudaStream_t);
    int (*gate_up)(const void*, const int*, const void*, void*, int, int, int, int, int, int, cudaStream_t);
    int (*down_combine)(const void*, const int*, const float*, const void*, int, const void*, void*, int, int, int, int, int, int,
                        float*, int, cudaStream_t);
    long long (*down_scratch_floats)(int, int, int, int, int);
    int (*sort_pairs)(const int*, int, int, int, int*, int*, int*, cudaStream_t);
    int (*combine)(const float*, const int*, const float*, const int*, const void*, void*, int, int, int, int, cudaStream_t);
    int (*route_scored)(const float*, int, int, int, int, const void*, int, int, int, float, int*, float*, float*, cudaStream_t);
};
struct AttentionTalk {
    last_error_fn last_error;
    int (*store)(void*, int, int, int, int, int, int, const int*, const int*, void*, void*, const int*, int, int, int, int, const void*,
                 const void*, int, void*, cudaStream_t);
    long long (*scratch_floats)(int, int, int, int, int);
    int (*rows)(const void*, int, const void*, const void*, const int*, int, int, const int*, const int*, int, int, int, int, int, int, int,
                float, const float*, const void*, int, const void*, int, void*, float*, int, cudaStream_t);
    long long (*prompt_scratch_floats)(int, int, int, int, int, int);
    int (*prompt)(const void*, int, const void*, const void*, const int*, int, int, const int*, const int*, const int*, int, int, int, int,
                  int, int, int, int, int, float, const float*, const void*, int, const void*, int, void*, float*, cudaStream_t);
};
struct AttentionMma {
    last_error_fn last_error;
    int (*run)(const void*, int, void*, const void*, const void*, int, const int*, int, int, const int*, const int*,
               const int*, const int*, int, int, int, int, int, int, int, float, int, int, float*, int*, int, int*,
               cudaStream_t);
    int (*clusters_at_once)(int, int);
};
struct AttentionTc {
    last_error_fn last_error;
    int (*run)(const void*, int, int, void*, const void*, const void*, int, const int*, int, const int*, const int*,
               const int*, const int*, int, int, int, int, int, int, float, int*, cudaStream_t);
};
struct Sampling {
    last_error_fn last_error;
    int (*sample)(const float*, int, int, int, const float*, const int*, const int*, unsigned long long, const int*, int*,
                  cudaStream_t);
};

const Rowwise& rowwise();
const GemmSimt& gemm_simt();
const GemmTc& gemm_tc();
const AttentionSimt& attention_simt();
const AttentionMma& attention_mma();
const AttentionTc& attention_tc();
const Sampling& sampling();
const AttentionWindow& attention_window();
const Residual& residual();
const Recurrence& recurrence();
const Routed& routed();
const Delta& delta();
const AttentionLatent& attention_latent();
const AttentionTalk& attention_talk();
const AttentionPooled& attention_pooled();

// Called with a family's name when its library is missing; returns 0 when it has built it.
typedef int (*builder_fn)(const char* family);
void set_builder(builder_fn f);
std::string library_dir();
std::string loaded_libraries();     // paths, one per line

}  // namespace kernels
}  // namespace friday
