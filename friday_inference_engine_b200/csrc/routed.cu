// Routed experts: the choice, and the experts' products for few rows.
//
//   route            per row: the `top` largest of the router's logits (the lower index wins a tie), their weights
//                    (softmax over the chosen logits only, or over all of them), optionally a dense map
//                    [rows][experts] that holds each chosen expert's weight and zero elsewhere
//   scale_by_route   act [rows][experts * inner] *= dense[row][column / inner]: after it, one product over all
//                    experts' down matrices side by side sums exactly the chosen experts
//   gate_up          for every (row, choice): act = silu(Wg_e h) * (Wu_e h), expert e's rows read where they lie
//   down_combine     out[row] = residual[row] + sum over choices of weight * (Wd_e act)
//
// gate_up and down_combine read only the chosen experts' weights, once per (row, choice): the form for one-token
// steps, where those bytes are the cost.  With many rows the dense form (all experts through the tensor-core
// product, scale_by_route, one down product) does more arithmetic but runs on the tensor cores.
//
// Router logits, the choice and the weights are fp32.  Gate and up weights are stored row by row in turn
// (gate 0, up 0, gate 1, ...), expert after expert: [experts * 2 * inner][width]; down: [width][experts * inner].
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* routed_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

constexpr int ROUTE_PER_LANE = 8;          // up to 256 experts

__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, int ld, int rows, int experts, int top, int softmax_all, int* __restrict__ ids,
             float* __restrict__ weights, float* __restrict__ dense) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= rows) return;
    float z[ROUTE_PER_LANE];
    float all_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        z[i] = e < experts ? logits[(size_t)row * ld + e] : -INFINITY;
        all_max = fmaxf(all_max, z[i]);
    }
    all_max = fr_warp_max(all_max);
    float all_sum = 0.f;
    if (softmax_all) {
#pragma unroll
        for (int i = 0; i < ROUTE_PER_LANE; ++i)
            if (lane + 32 * i < experts) all_sum += expf(z[i] - all_max);
        all_sum = fr_warp_sum(all_sum);
    }
    if (dense != nullptr)
        for (int e = lane; e < experts; e += 32) dense[(size_t)row * experts + e] = 0.f;
    __syncwarp();
    float first = 0.f, chosen_sum = 0.f;
    float my_logit = 0.f;                   // lane t keeps the t-th choice
    int my_id = -1;
    for (int t = 0; t < top; ++t) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < ROUTE_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < experts && (z[i] > best || (z[i] == best && e < best_e))) {
                best = z[i];
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        if (best_e >= experts) best_e = -1;          // no finite logit left (a dead row's garbage)
        if (t == 0) first = best;
        chosen_sum += expf(best - first);
        if (lane == (t & 31)) {
            my_logit = best;
            my_id = best_e;
        }
#pragma unroll
        for (int i = 0; i < ROUTE_PER_LANE; ++i)
            if (lane + 32 * i == best_e) z[i] = -INFINITY;
    }
    if (lane < top) {
        const float w = softmax_all ? expf(my_logit - all_max) / all_sum : expf(my_logit - first) / chosen_sum;
        ids[(size_t)row * top + lane] = my_id;
        weights[(size_t)row * top + lane] = w;
        if (dense != nullptr && my_id >= 0) dense[(size_t)row * experts + my_id] = w;
    }
}

// one row per blockIdx.y; eight consecutive channels per thread where rows allow 16-byte pieces
template <typename T>
__global__ void scale_by_route_kernel(T* __restrict__ act, const float* __restrict__ dense, int rows, int experts, int inner, int by_eight) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int per_row = experts * inner;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    T* a = act + (size_t)row * per_row;
    const float* d = dense + (size_t)row * experts;
    if (by_eight) {
        if constexpr (sizeof(T) == 2) {
            for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8; c < per_row; c += gridDim.x * blockDim.x * 8) {
                const float w = d[c / inner];
                uint4 v = *(const uint4*)(a + c);
                if (w == 0.f) v = make_uint4(0, 0, 0, 0);
                else {
                    __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(h[i]);
                        h[i] = __floats2bfloat162_rn(f.x * w, f.y * w);
                    }
                }
                *(uint4*)(a + c) = v;
            }
            continue;
        }
    }
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < per_row; c += gridDim.x * blockDim.x)
        fr_store(a + c, fr_load(a + c) * d[c / inner]);
  }
}

// block: one (row, choice) and a tile of `inner`; a warp per inner channel, lanes over the width
template <typename T>
__global__ void __launch_bounds__(256)
gate_up_kernel(const T* __restrict__ h, const int* __restrict__ ids, const T* __restrict__ w_gate_up, T* __restrict__ act,
               int top, int width, int inner, int per_block) {
    extern __shared__ float hs[];             // [width]
    fr_pdl_wait();
    fr_pdl_launch();
    const int pair = blockIdx.x;              // row * top + choice
    const int row = pair / top;
    const int e = ids[pair];
    for (int c = threadIdx.x; c < width; c += blockDim.x) hs[c] = fr_load(h + (size_t)row * width + c);
    __syncthreads();
    if (e < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.y * per_block;
    const T* w = w_gate_up + (size_t)e * 2 * inner * width;
    for (int f = f0 + warp; f < min(f0 + per_block, inner); f += 8) {
        const T* g = w + (size_t)(2 * f) * width;
        const T* u = g + width;
        float sg = 0.f, su = 0.f;
        for (int c = lane; c < width; c += 32) {
            sg = fmaf(hs[c], fr_load(g + c), sg);
            su = fmaf(hs[c], fr_load(u + c), su);
        }
        sg = fr_warp_sum(sg);
        su = fr_warp_sum(su);
        if (lane == 0) fr_store(act + (size_t)pair * inner + f, sg / (1.0f + expf(-sg)) * su);
    }
}

// Few rows: a block owns one expert and a tile of `inner`; it gathers the rows that chose the expert (at most MAX_SHARE,
// staged in shared memory in their own dtype) and reads every weight row once for all of them, 16 bytes per lane.
constexpr int MAX_SHARE = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gate_up_by_expert_kernel(const T* __restrict__ h, const int* __restrict__ ids, const T* __restrict__ w_gate_up, T* __restrict__ act,
                         int rows, int top, int width, int inner, int per_block) {
    extern __shared__ __align__(16) unsigned char raw[];
    T* hs = (T*)raw;                           // [MAX_SHARE][width]
    __shared__ int pairs[MAX_SHARE];
    __shared__ int n_pairs;
    constexpr int PER = 16 / sizeof(T);
    fr_pdl_wait();
    fr_pdl_launch();
    const int e = blockIdx.x;
    // the pairs that chose this expert, in order: the ids are read side by side, then one thread lists the matches
    __shared__ int chosen[MAX_SHARE * 32];
    for (int pr = threadIdx.x; pr < rows * top; pr += blockDim.x) chosen[pr] = ids[pr];
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0;
        for (int pr = 0; pr < rows * top && n < MAX_SHARE; ++pr)
            if (chosen[pr] == e) pairs[n++] = pr;
        n_pairs = n;
    }
    __syncthreads();
    const int n = n_pairs;
    if (n == 0) return;
    for (int idx = threadIdx.x; idx < n * (width / PER); idx += blockDim.x) {
        const int r = idx / (width / PER), c = idx % (width / PER);
        ((uint4*)(hs + (size_t)r * width))[c] = ((const uint4*)(h + (size_t)(pairs[r] / top) * width))[c];
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.y * per_block;
    const T* w = w_gate_up + (size_t)e * 2 * inner * width;
    for (int f = f0 + warp; f < min(f0 + per_block, inner); f += 8) {
        const uint4* g4 = (const uint4*)(w + (size_t)(2 * f) * width);
        const uint4* u4 = (const uint4*)(w + (size_t)(2 * f + 1) * width);
        float sg[MAX_SHARE], su[MAX_SHARE];
#pragma unroll
        for (int r = 0; r < MAX_SHARE; ++r) sg[r] = su[r] = 0.f;
        for (int c0 = lane; c0 < width / PER; c0 += 32 * 4) {
            uint4 gv[4], uv[4];                   // four pieces of each row in flight
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int c = c0 + 32 * k;
                if (c < width / PER) {
                    gv[k] = __ldg(g4 + c);
                    uv[k] = __ldg(u4 + c);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int c = c0 + 32 * k;
                if (c >= width / PER) break;
                float gf[PER], uf[PER];
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    gf[i] = fr_load((const T*)&gv[k] + i);
                    uf[i] = fr_load((const T*)&uv[k] + i);
                }
#pragma unroll
                for (int r = 0; r < MAX_SHARE; ++r) {
                    if (r < n) {
                        const uint4 hv = ((const uint4*)(hs + (size_t)r * width))[c];
#pragma unroll
                        for (int i = 0; i < PER; ++i) {
                            const float x = fr_load((const T*)&hv + i);
                            sg[r] = fmaf(x, gf[i], sg[r]);
                            su[r] = fmaf(x, uf[i], su[r]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MAX_SHARE; ++r) {
            if (r < n) {
                const float a = fr_warp_sum(sg[r]), b = fr_warp_sum(su[r]);
                if (lane == 0) fr_store(act + (size_t)pairs[r] * inner + f, a / (1.0f + expf(-a)) * b);
            }
        }
    }
}

// The same for the down product: a block owns one expert and a tile of output columns, stages the activations of the
// (row, choice) pairs that chose the expert, reads every weight row once for all of them and leaves each pair's part
// [pairs][width] in fp32; combine_kernel then adds the parts to the residual in the order of the choices, so the sum
// does not depend on which block finished first.
template <typename T>
__global__ void __launch_bounds__(256)
down_by_expert_kernel(const T* __restrict__ act, const int* __restrict__ ids, const T* __restrict__ w_down, int ld_down,
                      float* __restrict__ part, int rows, int top, int width, int inner, int per_block) {
    extern __shared__ __align__(16) unsigned char raw[];
    T* as = (T*)raw;                           // [MAX_SHARE][inner]
    __shared__ int pairs[MAX_SHARE];
    __shared__ int n_pairs;
    constexpr int PER = 16 / sizeof(T);
    fr_pdl_wait();
    fr_pdl_launch();
    const int e = blockIdx.x;
    // the pairs that chose this expert, in order: the ids are read side by side, then one thread lists the matches
    __shared__ int chosen[MAX_SHARE * 32];
    for (int pr = threadIdx.x; pr < rows * top; pr += blockDim.x) chosen[pr] = ids[pr];
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0;
        for (int pr = 0; pr < rows * top && n < MAX_SHARE; ++pr)
            if (chosen[pr] == e) pairs[n++] = pr;
        n_pairs = n;
    }
    __syncthreads();
    const int n = n_pairs;
    if (n == 0) return;
    for (int idx = threadIdx.x; idx < n * (inner / PER); idx += blockDim.x) {
        const int r = idx / (inner / PER), c = idx % (inner / PER);
        ((uint4*)(as + (size_t)r * inner))[c] = ((const uint4*)(act + (size_t)pairs[r] * inner))[c];
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = blockIdx.y * per_block;
    for (int col = c0 + warp; col < min(c0 + per_block, width); col += 8) {
        const uint4* w4 = (const uint4*)(w_down + (size_t)col * ld_down + (size_t)e * inner);
        float acc[MAX_SHARE];
#pragma unroll
        for (int r = 0; r < MAX_SHARE; ++r) acc[r] = 0.f;
        for (int f0 = lane; f0 < inner / PER; f0 += 32 * 4) {
            uint4 wv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (f0 + 32 * k < inner / PER) wv[k] = __ldg(w4 + f0 + 32 * k);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int f = f0 + 32 * k;
                if (f >= inner / PER) break;
                float wf[PER];
#pragma unroll
                for (int i = 0; i < PER; ++i) wf[i] = fr_load((const T*)&wv[k] + i);
#pragma unroll
                for (int r = 0; r < MAX_SHARE; ++r) {
                    if (r < n) {
                        const uint4 av = ((const uint4*)(as + (size_t)r * inner))[f];
#pragma unroll
                        for (int i = 0; i < PER; ++i) acc[r] = fmaf(fr_load((const T*)&av + i), wf[i], acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MAX_SHARE; ++r) {
            if (r < n) {
                const float v = fr_warp_sum(acc[r]);
                if (lane == 0) part[(size_t)pairs[r] * width + col] = v;
            }
        }
    }
}

// part: one row per (row, choice) pair, at the pair's own index or, with `pos`, at pos[pair] (pairs sorted by expert)
template <typename TR>
__global__ void combine_kernel(const float* __restrict__ part, const int* __restrict__ ids, const float* __restrict__ weights,
                               const int* __restrict__ pos, const TR* __restrict__ residual, TR* __restrict__ out, int rows, int top,
                               int width) {
    fr_pdl_wait();
    fr_pdl_launch();
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const size_t pair = (size_t)row * top + j;
            if (ids[pair] >= 0) total = fmaf(weights[pair], part[(size_t)(pos != nullptr ? pos[pair] : (int)pair) * width + c], total);
        }
        const float r = residual != nullptr ? fr_load(residual + (size_t)row * width + c) : 0.f;
        fr_store(out + (size_t)row * width + c, r + total);
    }
  }
}

// The (row, choice) pairs in the order of their experts: offsets[e] .. offsets[e + 1] are expert e's places, pos[pair] the
// pair's place, row_at[place] the row whose activations belong there.  Which of an expert's places a pair gets depends on
// scheduling; no result depends on it, since every place is computed from its own row alone.  One block.
__global__ void __launch_bounds__(1024) sort_pairs_kernel(const int* __restrict__ ids, int n_pairs, int top, int experts,
                                                          int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ row_at) {
    __shared__ int cnt[256], off[257], cur[256];
    fr_pdl_wait();
    fr_pdl_launch();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = cur[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            off[e] = at;
            at += cnt[e];
        }
        off[experts] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = off[e];
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) {
            const int place = off[e] + atomicAdd(&cur[e], 1);
            pos[p] = place;
            row_at[place] = p / top;
        } else {
            pos[p] = 0;
        }
    }
}

// block: one row and a tile of the width; a warp per output column, lanes over inner
template <typename T, typename TR>
__global__ void __launch_bounds__(256)
down_combine_kernel(const T* __restrict__ act, const int* __restrict__ ids, const float* __restrict__ weights,
                    const T* __restrict__ w_down, int ld_down, const TR* __restrict__ residual, TR* __restrict__ out, int top,
                    int width, int inner, int per_block) {
    extern __shared__ float as[];             // [top][inner]
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    for (int i = threadIdx.x; i < top * inner; i += blockDim.x) as[i] = fr_load(act + (size_t)row * top * inner + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = blockIdx.y * per_block;
    for (int c = c0 + warp; c < min(c0 + per_block, width); c += 8) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = ids[(size_t)row * top + j];
            if (e < 0) continue;
            const T* w = w_down + (size_t)c * ld_down + (size_t)e * inner;
            float s = 0.f;
            constexpr int PER = 16 / sizeof(T);
            if (inner % PER == 0 && (((uintptr_t)w) & 15) == 0) {
                for (int f = lane * PER; f < inner; f += 32 * PER) {
                    const uint4 wv = *(const uint4*)(w + f);
#pragma unroll
                    for (int i = 0; i < PER; ++i) s = fmaf(as[j * inner + f + i], fr_load((const T*)&wv + i), s);
                }
            } else {
                for (int f = lane; f < inner; f += 32) s = fmaf(as[j * inner + f], fr_load(w + f), s);
            }
            total = fmaf(weights[(size_t)row * top + j], fr_warp_sum(s), total);
        }
        if (lane == 0) {
            const float r = residual != nullptr ? fr_load(residual + (size_t)row * width + c) : 0.f;
            fr_store(out + (size_t)row * width + c, r + total);
        }
    }
}

// Channels (of the inner size, or of the width) that a block of the by-expert kernels owns; FRIDAY_EXPERT_TILE overrides
// (a multiple of 8, for measurements: 8 to 64 differ by less than a tenth).
inline int expert_tile() {
    static int v = 0;
    if (v == 0) {
        const char* e = getenv("FRIDAY_EXPERT_TILE");
        const int t = e ? atoi(e) : 0;
        v = (t >= 8 && t <= 256 && t % 8 == 0) ? t : 16;
    }
    return v;
}

}  // namespace

FR_EXPORT int routed_route(const float* logits, int ld, int rows, int experts, int top, int softmax_all, int* ids, float* weights,
                           float* dense, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (experts < 1 || experts > 32 * ROUTE_PER_LANE) FR_REFUSE("route: %d experts (1 to %d)", experts, 32 * ROUTE_PER_LANE);
    if (top < 1 || top > experts || top > 32) FR_REFUSE("route: top %d of %d experts (at most 32)", top, experts);
    FR_CUDA(fr_launch(route_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, logits, ld, rows, experts, top, softmax_all, ids,
                      weights, dense));
    FR_CHECK_LAUNCH("route");
    return FR_OK;
}

FR_EXPORT int routed_scale_by_route(void* act, const float* dense, int rows, int experts, int inner, int dtype, cudaStream_t stream) {
    if (rows <= 0 || experts <= 0 || inner <= 0) return FR_OK;
    const long long per_row = (long long)experts * inner;
    if (per_row > 0x7fffffffLL) FR_REFUSE("scale_by_route: %lld channels per row", per_row);
    const int by_eight = dtype == FR_BF16 && inner % 8 == 0 && (((uintptr_t)act) & 15) == 0;
    const long long items = by_eight ? per_row / 8 : per_row;
    const int bx = (int)((items + 255) / 256 < 64 ? (items + 255) / 256 : 64);
    if (dtype == FR_F32) FR_CUDA(fr_launch(scale_by_route_kernel<float>, dim3(bx, rows < 65535 ? rows : 65535), dim3(256), 0, stream, (float*)act, dense, rows, experts, inner, 0));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(scale_by_route_kernel<bf16>, dim3(bx, rows < 65535 ? rows : 65535), dim3(256), 0, stream, (bf16*)act, dense, rows, experts, inner, by_eight));
    else FR_REFUSE("scale_by_route: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("scale_by_route");
    return FR_OK;
}

FR_EXPORT int routed_gate_up(const void* h, const int* ids, const void* w_gate_up, void* act, int rows, int top, int experts, int width,
                             int inner, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) FR_REFUSE("gate_up: width %d does not fit an SM's shared memory", width);
    const int per_block = inner < 64 ? inner : 64;
    const dim3 grid(rows * top, (inner + per_block - 1) / per_block);
    if (grid.y > 65535) FR_REFUSE("gate_up: inner size %d", inner);
    // few rows: one block per (expert, tile) reads the weights once for all rows that chose the expert
    const size_t esize = dtype == FR_F32 ? 4 : 2;
    const size_t share = (size_t)(rows < MAX_SHARE ? rows : MAX_SHARE) * width * esize;     // rows that can choose one expert
    if (dtype == FR_BF16 && rows <= MAX_SHARE && experts > 0 && width % (16 / esize) == 0 && share <= 160 * 1024 &&
        ((((uintptr_t)h) | ((uintptr_t)w_gate_up)) & 15) == 0) {
        const int eper = expert_tile();          // inner channels per block: enough blocks to fill the device
        const dim3 eg(experts, (inner + eper - 1) / eper);
        if (share > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(gate_up_by_expert_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)share));
        FR_CUDA(fr_launch(gate_up_by_expert_kernel<bf16>, eg, dim3(256), share, stream, (const bf16*)h, ids, (const bf16*)w_gate_up,
                          (bf16*)act, rows, top, width, inner, eper));
        FR_CHECK_LAUNCH("gate_up (by expert)");
        return FR_OK;
    }
    if (dtype == FR_F32) {
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(gate_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(gate_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, ids, (const float*)w_gate_up,
                          (float*)act, top, width, inner, per_block));
    } else if (dtype == FR_BF16) {
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(gate_up_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(gate_up_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)h, ids, (const bf16*)w_gate_up,
                          (bf16*)act, top, width, inner, per_block));
    } else {
        FR_REFUSE("gate_up: unknown dtype %d", dtype);
    }
    FR_CHECK_LAUNCH("gate_up");
    return FR_OK;
}

// Floats of scratch that routed_down_combine wants for these sizes (0: none).
FR_EXPORT long long routed_down_scratch_floats(int rows, int top, int width, int inner, int dtype) {
    const size_t share = (size_t)(rows < MAX_SHARE ? rows : MAX_SHARE) * inner * 2;
    if (dtype == FR_BF16 && rows <= MAX_SHARE && inner % 8 == 0 && share <= 160 * 1024) return (long long)rows * top * width;
    return 0;
}

// residual and out [rows][width] in res_dtype (fp32 for a 32-bit residual stream); residual may be null.
FR_EXPORT int routed_down_combine(const void* act, const int* ids, const float* weights, const void* w_down, int ld_down,
                                  const void* residual, void* out, int res_dtype, int rows, int top, int experts, int width, int inner,
                                  float* scratch, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (scratch != nullptr && routed_down_scratch_floats(rows, top, width, inner, dtype) > 0 && experts > 0 && ld_down % 8 == 0 &&
        ((((uintptr_t)act) | ((uintptr_t)w_down)) & 15) == 0 && rows <= 65535) {
        const size_t share = (size_t)(rows < MAX_SHARE ? rows : MAX_SHARE) * inner * 2;
        const int per = expert_tile();
        if (share > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(down_by_expert_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)share));
        FR_CUDA(fr_launch(down_by_expert_kernel<bf16>, dim3(experts, (width + per - 1) / per), dim3(256), share, stream, (const bf16*)act, ids,
                          (const bf16*)w_down, ld_down, scratch, rows, top, width, inner, per));
        FR_CHECK_LAUNCH("down (by expert)");
        const dim3 cg((width + 255) / 256, rows);
        if (res_dtype == FR_F32) FR_CUDA(fr_launch(combine_kernel<float>, cg, dim3(256), 0, stream, (const float*)scratch, ids, weights,
                                                   (const int*)nullptr, (const float*)residual, (float*)out, rows, top, width));
        else if (res_dtype == FR_BF16) FR_CUDA(fr_launch(combine_kernel<bf16>, cg, dim3(256), 0, stream, (const float*)scratch, ids, weights,
                                                         (const int*)nullptr, (const bf16*)residual, (bf16*)out, rows, top, width));
        else FR_REFUSE("down_combine: unknown residual dtype %d", res_dtype);
        FR_CHECK_LAUNCH("combine");
        return FR_OK;
    }
    const size_t smem = (size_t)top * inner * sizeof(float);
    if (smem > 200 * 1024) FR_REFUSE("down_combine: top %d x inner %d does not fit an SM's shared memory", top, inner);
    const int per_block = width < 64 ? width : 64;
    const dim3 grid(rows, (width + per_block - 1) / per_block);
    if (grid.y > 65535) FR_REFUSE("down_combine: width %d", width);
#define DOWN(T, TR)                                                                                                             \
    do {                                                                                                                        \
        if (smem > 48 * 1024)                                                                                                   \
            FR_CUDA(cudaFuncSetAttribute(down_combine_kernel<T, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  \
        FR_CUDA(fr_launch(down_combine_kernel<T, TR>, grid, dim3(256), smem, stream, (const T*)act, ids, weights, (const T*)w_down, \
                          ld_down, (const TR*)residual, (TR*)out, top, width, inner, per_block));                               \
    } while (0)
    if (dtype == FR_F32 && res_dtype == FR_F32) DOWN(float, float);
    else if (dtype == FR_BF16 && res_dtype == FR_F32) DOWN(bf16, float);
    else if (dtype == FR_BF16 && res_dtype == FR_BF16) DOWN(bf16, bf16);
    else FR_REFUSE("down_combine: no kernel for dtypes %d and %d", dtype, res_dtype);
#undef DOWN
    FR_CHECK_LAUNCH("down_combine");
    return FR_OK;
}

// offsets [experts + 1], pos [rows * top], row_at [rows * top]: see sort_pairs_kernel.
FR_EXPORT int routed_sort_pairs(const int* ids, int rows, int top, int experts, int* offsets, int* pos, int* row_at, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (experts < 1 || experts > 256) FR_REFUSE("sort_pairs: %d experts (1 to 256)", experts);
    FR_CUDA(fr_launch(sort_pairs_kernel, dim3(1), dim3(1024), 0, stream, ids, rows * top, top, experts, offsets, pos, row_at));
    FR_CHECK_LAUNCH("sort_pairs");
    return FR_OK;
}

// out [rows][width] = residual + sum over a row's choices of weight * part[pos[pair]]
FR_EXPORT int routed_combine(const float* part, const int* ids, const float* weights, const int* pos, const void* residual, void* out,
                             int res_dtype, int rows, int top, int width, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    const dim3 cg((width + 255) / 256, rows < 65535 ? rows : 65535);
    if (res_dtype == FR_F32) FR_CUDA(fr_launch(combine_kernel<float>, cg, dim3(256), 0, stream, part, ids, weights, pos, (const float*)residual,
                                               (float*)out, rows, top, width));
    else if (res_dtype == FR_BF16) FR_CUDA(fr_launch(combine_kernel<bf16>, cg, dim3(256), 0, stream, part, ids, weights, pos,
                                                     (const bf16*)residual, (bf16*)out, rows, top, width));
    else FR_REFUSE("combine: unknown residual dtype %d", res_dtype);
    FR_CHECK_LAUNCH("combine");
    return FR_OK;
}

// ------------------------------------------------------------------ a choice by biased sigmoid scores among groups of experts
// Per row: s_e = sigmoid(z_e) and c_e = s_e + bias_e (bias null: c = s).  Experts e with the same e / (experts / groups)
// are one group, ranked by r = the two largest c of the group added up (one c, if a group is a single expert).  Outside
// the `keep` groups of highest r an expert cannot win (its c reads as -inf, so negative c inside still beat it).  The `top`
// experts of highest c win (ties: the lower index, for groups and experts alike) with weight s_e * scale; the weights are
// left as they are, they need not sum to one.  fp32.
namespace {

__global__ void __launch_bounds__(128)
route_scored_kernel(const float* __restrict__ logits, int ld, int rows, int experts, int top, FrVec bias, int groups, int keep,
                    float scale, int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ dense) {
    __shared__ float s_all[4][32 * ROUTE_PER_LANE], c_all[4][32 * ROUTE_PER_LANE], g_all[4][32 * ROUTE_PER_LANE];
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= rows) return;
    float* s = s_all[warp];
    float* c = c_all[warp];
    float* gs = g_all[warp];
    for (int e = lane; e < experts; e += 32) {
        const float v = 1.0f / (1.0f + expf(-logits[(size_t)row * ld + e]));
        s[e] = v;
        c[e] = bias.p != nullptr ? v + bias.at(e) : v;
        if (dense != nullptr) dense[(size_t)row * experts + e] = 0.f;
    }
    __syncwarp();
    if (groups > 1) {
        const int size = experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;          // the two largest of the group
            for (int i = 0; i < size; ++i) {
                const float v = c[g * size + i];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gs[g] = size > 1 ? a + b : a;
        }
        __syncwarp();
        for (int g = lane; g < groups; g += 32) {
            int better = 0;
            for (int o = 0; o < groups; ++o) better += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
            if (better >= keep)
                for (int i = 0; i < size; ++i) c[g * size + i] = -INFINITY;
        }
        __syncwarp();
    }
    float z[ROUTE_PER_LANE];
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) z[i] = lane + 32 * i < experts ? c[lane + 32 * i] : -INFINITY;
    int my_id = -1;
    for (int t = 0; t < top; ++t) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < ROUTE_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < experts && (z[i] > best || (z[i] == best && e < best_e))) {
                best = z[i];
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        if (best_e >= experts || best == -INFINITY) best_e = -1;          // nothing left that may be chosen
        if (lane == (t & 31)) my_id = best_e;
#pragma unroll
        for (int i = 0; i < ROUTE_PER_LANE; ++i)
            if (lane + 32 * i == best_e) z[i] = -INFINITY;
    }
    if (lane < top) {
        const float w = my_id >= 0 ? s[my_id] * scale : 0.f;
        ids[(size_t)row * top + lane] = my_id;
        weights[(size_t)row * top + lane] = w;
        if (dense != nullptr && my_id >= 0) dense[(size_t)row * experts + my_id] = w;
    }
}

}  // namespace

FR_EXPORT int routed_route_scored(const float* logits, int ld, int rows, int experts, int top, const void* bias, int bias_dtype, int groups,
                                  int keep, float scale, int* ids, float* weights, float* dense, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (experts < 1 || experts > 32 * ROUTE_PER_LANE) FR_REFUSE("route: %d experts (1 to %d)", experts, 32 * ROUTE_PER_LANE);
    if (top < 1 || top > experts || top > 32) FR_REFUSE("route: top %d of %d experts (at most 32)", top, experts);
    if (groups < 1 || experts % groups || keep < 1 || keep > groups) FR_REFUSE("route: %d experts in %d groups, %d kept", experts, groups, keep);
    FR_CUDA(fr_launch(route_scored_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, logits, ld, rows, experts, top,
                      FrVec{bias, bias_dtype}, groups, keep, scale, ids, weights, dense));
    FR_CHECK_LAUNCH("route_scored");
    return FR_OK;
}
