// Opens the kernel libraries and resolves their entry points (kernels.h).
#include "ops/kernels.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <sys/stat.h>

#include <map>
#include <mutex>

#include "friday/base.h"

namespace friday {
namespace kernels {

namespace {
std::mutex g_mutex;
builder_fn g_builder = nullptr;
std::map<std::string, void*> g_handles;
std::map<std::string, std::string> g_paths;

bool exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

void* open_family(const std::string& family) {
    auto it = g_handles.find(family);
    if (it != g_handles.end()) return it->second;
    // The builder decides whether the library on disk was made from the present sources.
    if (g_builder && g_builder(family.c_str()) != 0)
        throw KernelError("the kernel library '" + family + "' could not be built (see the builder's message above)");
    const std::string path = library_dir() + "/libfriday_" + family + ".so";
    if (!exists(path))
        throw KernelError("kernel library " + path + " is missing and nothing is set up to build it: run "
                          "`python -m friday_inference_engine_b200.ops.build` (needs nvcc), or set FRIDAY_BUILD_DIR "
                          "to the folder that holds the built libraries; there is no other path");
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) throw KernelError("cannot load " + path + ": " + dlerror());
    g_handles[family] = h;
    g_paths[family] = path;
    return h;
}

template <class F> void resolve(void* h, const std::string& family, const char* name, F& out) {
    void* s = dlsym(h, name);
    if (!s) throw KernelError("kernel library '" + family + "' has no entry point " + name);
    out = (F)s;
}
}  // namespace

void set_builder(builder_fn f) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_builder = f;
}

std::string library_dir() {
    const char* env = getenv("FRIDAY_BUILD_DIR");
    if (env && env[0]) return env;
    Dl_info info;
    if (dladdr((void*)&library_dir, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t slash = p.rfind('/');
        return slash == std::string::npos ? "." : p.substr(0, slash);
    }
    return ".";
}

std::string loaded_libraries() {
    std::lock_guard<std::mutex> lock(g_mutex);
    std::string out;
    for (const auto& kv : g_paths) out += kv.second + "\n";
    return out;
}

#define FAMILY(Type, fn, family, ...)                          \
    const Type& fn() {                                         \
        static Type t;                                         \
        static bool ready = false;                             \
        std::lock_guard<std::mutex> lock(g_mutex);             \
        if (!ready) {                                          \
            void* h = open_family(family);                     \
            const std::string fam = family;                    \
            resolve(h, fam, family "_last_error", t.last_error); \
            __VA_ARGS__                                        \
            ready = true;                                      \
        }                                                      \
        return t;                                              \
    }

FAMILY(Rowwise, rowwise, "rowwise",
       resolve(h, fam, "rowwise_embedding", t.embedding); resolve(h, fam, "rowwise_gather_rows", t.gather_rows);
       resolve(h, fam, "rowwise_rmsnorm", t.rmsnorm); resolve(h, fam, "rowwise_swiglu", t.swiglu);
       resolve(h, fam, "rowwise_gated_act", t.gated_act);
       resolve(h, fam, "rowwise_rope_kv_write", t.rope_kv_write); resolve(h, fam, "rowwise_advance", t.advance);
       resolve(h, fam, "rowwise_scale_rows", t.scale_rows); resolve(h, fam, "rowwise_finish_logits", t.finish_logits);
       resolve(h, fam, "rowwise_random_normal", t.random_normal);)
FAMILY(GemmSimt, gemm_simt, "gemm_simt", resolve(h, fam, "gemm_simt", t.gemm);)
FAMILY(GemmTc, gemm_tc, "gemm_tc", resolve(h, fam, "gemm_tc_fused", t.fused); resolve(h, fam, "gemm_tc_plan", t.plan);)
FAMILY(AttentionSimt, attention_simt, "attention_simt", resolve(h, fam, "attention_simt", t.run);
       resolve(h, fam, "attention_simt_masked", t.masked);)
FAMILY(AttentionWindow, attention_window, "attention_window", resolve(h, fam, "attention_window_fits", t.fits);
       resolve(h, fam, "attention_window", t.run);)
FAMILY(Residual, residual, "residual", resolve(h, fam, "residual_norm_cast", t.norm_cast);
       resolve(h, fam, "residual_concat_cast", t.concat_cast); resolve(h, fam, "residual_add_scaled", t.add_scaled);
       resolve(h, fam, "residual_kv_store", t.kv_store); resolve(h, fam, "residual_token_input", t.token_input);
       resolve(h, fam, "residual_gelu_table", t.gelu_table); resolve(h, fam, "residual_rms_add", t.rms_add);
       resolve(h, fam, "residual_layernorm_cast", t.layernorm_cast); resolve(h, fam, "residual_embed_rows", t.embed_rows);
       resolve(h, fam, "residual_embed_pos", t.embed_pos); resolve(h, fam, "residual_norm_shift", t.norm_shift);
       resolve(h, fam, "residual_post_norm_add", t.post_norm_add); resolve(h, fam, "residual_two_sided_act", t.two_sided_act);
       resolve(h, fam, "residual_embed_pair", t.embed_pair); resolve(h, fam, "residual_norm_conv", t.norm_conv);
       resolve(h, fam, "residual_norm_conv_state", t.norm_conv_state); resolve(h, fam, "residual_rms_pair_add", t.rms_pair_add);)
FAMILY(Recurrence, recurrence, "recurrence", resolve(h, fam, "recurrence_shift_mix", t.shift_mix);
       resolve(h, fam, "recurrence_tanh_rows", t.tanh_rows); resolve(h, fam, "recurrence_scan", t.scan);
       resolve(h, fam, "recurrence_scan_plan", t.scan_plan);
       resolve(h, fam, "recurrence_head_norm_gate", t.head_norm_gate);)
FAMILY(Routed, routed, "routed", resolve(h, fam, "routed_route", t.route);
       resolve(h, fam, "routed_scale_by_route", t.scale_by_route); resolve(h, fam, "routed_gate_up", t.gate_up);
       resolve(h, fam, "routed_down_combine", t.down_combine);
       resolve(h, fam, "routed_down_scratch_floats", t.down_scratch_floats);
       resolve(h, fam, "routed_sort_pairs", t.sort_pairs); resolve(h, fam, "routed_combine", t.combine);
       resolve(h, fam, "routed_route_scored", t.route_scored);)
FAMILY(AttentionTalk, attention_talk, "attention_talk", resolve(h, fam, "attention_talk_store", t.store);
       resolve(h, fam, "attention_talk_scratch_floats", t.scratch_floats); resolve(h, fam, "attention_talk_rows", t.rows);
       resolve(h, fam, "attention_talk_prompt_scratch_floats", t.prompt_scratch_floats);
       resolve(h, fam, "attention_talk_prompt", t.prompt);)
FAMILY(Delta, delta, "delta", resolve(h, fam, "delta_conv_prepare", t.conv_prepare);
       resolve(h, fam, "delta_conv_state", t.conv_state); resolve(h, fam, "delta_scan", t.scan);
       resolve(h, fam, "delta_general_prepare", t.general_prepare); resolve(h, fam, "delta_general_scan", t.general_scan);)
FAMILY(AttentionLatent, attention_latent, "attention_latent", resolve(h, fam, "attention_latent_rotate_pairs", t.rotate_pairs);
       resolve(h, fam, "attention_latent_prepare", t.prepare); resolve(h, fam, "attention_latent_head_linear", t.head_linear);
       resolve(h, fam, "attention_latent", t.run); resolve(h, fam, "attention_latent_gather", t.gather);
       resolve(h, fam, "attention_latent_softmax_split", t.softmax_split); resolve(h, fam, "attention_latent_gate_cast", t.gate_cast);
       resolve(h, fam, "attention_latent_key_concat", t.key_concat);)
FAMILY(AttentionPooled, attention_pooled, "attention_pooled", resolve(h, fam, "attention_pooled_prepare", t.prepare);
       resolve(h, fam, "attention_pooled_pool", t.pool); resolve(h, fam, "attention_pooled_scratch_floats", t.scratch_floats);
       resolve(h, fam, "attention_pooled_rows", t.rows); resolve(h, fam, "attention_pooled_prompt_fits", t.prompt_fits);
       resolve(h, fam, "attention_pooled_prompt", t.prompt);)
FAMILY(AttentionMma, attention_mma, "attention_mma", resolve(h, fam, "attention_mma", t.run);
       resolve(h, fam, "attention_mma_clusters_at_once", t.clusters_at_once);)
FAMILY(AttentionTc, attention_tc, "attention_tc", resolve(h, fam, "attention_tc", t.run);)
FAMILY(Sampling, sampling, "sampling", resolve(h, fam, "sampling_sample", t.sample);)

}  // namespace kernels
}  // namespace friday
