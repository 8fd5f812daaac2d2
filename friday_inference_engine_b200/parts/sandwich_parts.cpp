// A residual block with a norm on both sides of every sublayer, an optional token shift ahead of the mixer, and a dense
// feed-forward with a two-sided activation.
//
//   block "sandwich"       x <- x + m * norm1b(mixer(shift(norm1(x))));  x <- x + m * norm2b(ff(norm2(x)))  (the second if the
//                          block has a feed-forward).  m is "residual_mult".  With "shift" (a tensor [width], s) the mixer
//                          reads h + (h_before - h) * s, h_before being the row before's h (zeros before a sequence's first
//                          row); the h of a sequence's last row is kept as a state beside what the mixer asks of the cache.
//   feed_forward "dense"   Wd act(Wu h); "activation": "two_sided" with the tensor "act" = (p, q):
//                          z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2
//
// The stream is 32-bit; the norms, the shift and the sums are fp32 (csrc/residual.cu).  The sublayers return their results
// alone (they are handed an undefined residual), 32-bit, and the block sums: the norm after a sublayer, the sum and the norm
// ahead of the next sublayer are one kernel.
#include <math.h>

#include "friday/ops.h"
#include "friday/parts.h"

namespace friday {

class DenseFF : public FeedForward {
public:
    DenseFF(const PartSpec& s, const BuildEnv& e) : FeedForward(e) {
        inner_ = s.params.get_int("inner", 0);
        if (inner_ <= 0) throw ConfigError("dense feed-forward needs 'inner'");
        const std::string act = s.params.get_string("activation", "two_sided");
        if (act != "two_sided") throw ConfigError("dense feed-forward: activation '" + act + "' is not one it has (two_sided)");
        declare("up", {inner_, e.width});
        declare("down", {e.width, inner_});
        declare("act", {2});
    }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext&, Norm*) override {
        Tensor z = ops.linear(h, tensor("up"));
        ops.two_sided_act(z, tensor("act"));
        if (!residual.defined()) return PartOut(ops.linear(Rows(z), tensor("down"), nullptr, nullptr, (int)DType::F32));
        return PartOut(ops.linear_residual(Rows(z), tensor("down"), nullptr, residual));
    }

private:
    int64_t inner_;
};

class SandwichBlock : public Block {
public:
    SandwichBlock(const PartSpec& s, const BuildEnv& e) : Block(e) {
        mult_ = (float)s.params.get_double("residual_mult", 1.0);
        shift_name_ = s.params.get_string("shift", "");
        const PartSpec& mx = s.part("mixer");
        norm1_ = adopt(s.part("norm1").prefix, build<Norm>("norm", s.part("norm1"), e));
        norm1b_ = adopt(s.part("norm1b").prefix, build<Norm>("norm", s.part("norm1b"), e));
        mixer_ = adopt(mx.prefix, build<Mixer>("mixer", mx, e));
        if (s.parts.count("feed_forward")) {
            const PartSpec& ff = s.part("feed_forward");
            norm2_ = adopt(s.part("norm2").prefix, build<Norm>("norm", s.part("norm2"), e));
            norm2b_ = adopt(s.part("norm2b").prefix, build<Norm>("norm", s.part("norm2b"), e));
            ffn_ = adopt(ff.prefix, build<FeedForward>("feed_forward", ff, e));
        }
        if (!shift_name_.empty()) declare(shift_name_, {e.width});
    }
    CacheRequest cache_request() const override {
        if (shift_name_.empty()) return mixer_->cache_request();
        return CacheRequest::several({mixer_->cache_request(), CacheRequest::state({env.width}, DType::F32)});
    }

    PartOut forward(Ops& ops, const Tensor& x, const Rows*, const StepContext& ctx, const CacheView& view, Norm*) override {
        if (x.dtype != DType::F32) throw ConfigError("a sandwich block needs a 32-bit residual stream");
        Tensor w, wb;
        float eps = 0.f, epsb = 0.f;
        static const CacheView none;
        const CacheView* mixer_view = &view;
        Rows h;
        if (!shift_name_.empty()) {
            if (view.kind != CacheRequest::Several || view.parts.size() != 2)
                throw KernelError("sandwich block: the cache view does not have the mixer's part and the shift's");
            mixer_view = &view.parts[0];
            if (!norm1_->rms_parts(&w, &eps)) throw ConfigError("sandwich block: a token shift follows a plain RMS norm");
            h = Rows(ops.norm_shift(x, w, eps, tensor(shift_name_), view.parts[1], ctx, env.dtype));
        } else {
            h = Rows(norm1_->forward(ops, x));
        }
        Tensor y = mixer_->forward(ops, h, Tensor(), ctx, mixer_view->kind == CacheRequest::None ? none : *mixer_view, nullptr).x;
        if (!ffn_) return PartOut(after(ops, x, y, norm1b_, nullptr, nullptr));
        Tensor h2;
        Tensor mid = after(ops, x, y, norm1b_, norm2_, &h2);
        Tensor y2 = ffn_->forward(ops, Rows(h2), Tensor(), ctx, nullptr).x;
        return PartOut(after(ops, mid, y2, norm2b_, nullptr, nullptr));
    }

private:
    // x + m * post(y), and next(of that sum) if asked for; one kernel where both norms are plain RMS norms
    Tensor after(Ops& ops, const Tensor& x, const Tensor& y, Norm* post, Norm* next, Tensor* next_out) {
        Tensor w, w2;
        float eps = 0.f, eps2 = 0.f;
        const bool plain = post->rms_parts(&w, &eps) && (!next || next->rms_parts(&w2, &eps2));
        if (plain && y.dtype == DType::F32)
            return ops.post_norm_add(x, y, w, eps, mult_, next ? &w2 : nullptr, eps2, env.dtype, next_out);
        Tensor sum = ops.add_scaled(x, post->forward(ops, y), mult_);
        if (next) *next_out = next->forward(ops, sum);
        return sum;
    }

    float mult_;
    std::string shift_name_;
    Norm *norm1_ = nullptr, *norm1b_ = nullptr, *norm2_ = nullptr, *norm2b_ = nullptr;
    Mixer* mixer_ = nullptr;
    FeedForward* ffn_ = nullptr;
};

namespace {
PartRegistrar w1("feed_forward", "dense", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new DenseFF(s, e); });
PartRegistrar w2("block", "sandwich", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new SandwichBlock(s, e); });
}  // namespace

}  // namespace friday
