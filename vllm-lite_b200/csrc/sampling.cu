// Sampling of one token per row of float32 logits, on the device.
//
// Order of the steps, as in crates/core/src/sampling.rs:497-636 of the reference:
//   (1) repeat penalty   l >= 0 ? l / p : l * p    once per distinct seen id
//   (2) presence penalty l -= p                    once per distinct seen id
//   (3) logit bias       l[id] += b
//   (4) temperature      l /= T            (T > 0 and T != 1)
//   (5) top-k            the k-th largest value is the threshold, l < thr is dropped,
//                        ties at the threshold are kept
//   (6) T <= 0: argmax (ties: lowest index, NaN counts as -inf); else softmax with the
//       maximum subtracted; top_p < 1 keeps the most probable tokens, in descending
//       order, up to and including the one with which the cumulative probability
//       exceeds top_p; the draw is the inverse CDF at u over the kept tokens.
// Two choices are this engine's own.  The draw walks the kept tokens in index order
// (the reference walks nucleus tokens in sorted order): same distribution, other
// token for the same u.  Tokens whose probability equals the nucleus' last one are
// all kept.  Probabilities are accumulated as 40-bit fixed-point integers, so sums do
// not depend on the order in which threads add and a draw is reproducible.
//
// vl_apply_penalties works on ragged per-row lists; vl_sample uses one block of 1024
// threads per row.  Any vocabulary size.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_FIX 1099511627776.0f /* 2^40 */

__device__ __forceinline__ unsigned order_key(float v) {
    unsigned k = __float_as_uint(v);
    return (k & 0x80000000u) ? ~k : (k | 0x80000000u);
}
__device__ __forceinline__ float clean(float v, float inv_t) {
    v = v * inv_t;
    return (v != v) ? -INFINITY : v;
}

__global__ void apply_penalties_kernel(float* __restrict__ logits, long long row_stride, int V,
                                       const int* __restrict__ seen_off, const int* __restrict__ seen_ids,
                                       const float* __restrict__ repeat_p, const float* __restrict__ presence_p,
                                       const int* __restrict__ bias_off, const int* __restrict__ bias_ids,
                                       const float* __restrict__ bias_vals) {
    const int r = blockIdx.x;
    float* l = logits + (size_t)r * row_stride;
    if (seen_off) {
        const float rp = repeat_p ? repeat_p[r] : 1.f;
        const float pp = presence_p ? presence_p[r] : 0.f;
        for (int i = seen_off[r] + threadIdx.x; i < seen_off[r + 1]; i += blockDim.x) {
            const int id = seen_ids[i];          // the host passes each id once per row
            if (id < 0 || id >= V) continue;
            float v = l[id];
            if (rp != 1.f) v = v >= 0.f ? v / rp : v * rp;
            v -= pp;
            l[id] = v;
        }
    }
    __syncthreads();
    if (bias_off) {
        for (int i = bias_off[r] + threadIdx.x; i < bias_off[r + 1]; i += blockDim.x) {
            const int id = bias_ids[i];
            if (id >= 0 && id < V) l[id] += bias_vals[i];
        }
    }
}

struct ArgBest { float v; int i; };
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out_token, float* __restrict__ out_logprob) {
    __shared__ unsigned s_cnt[256];
    __shared__ unsigned long long s_mass[256];
    __shared__ float s_f[32];
    __shared__ int s_i[32];
    __shared__ unsigned long long s_w[32];
    __shared__ unsigned s_prefix, s_remaining;
    __shared__ unsigned long long s_above, s_total;
    __shared__ float s_max;
    __shared__ int s_pick;

    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* l = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.f / temp;
    int k = top_k ? top_k[r] : 0;
    const float tp = top_p ? top_p[r] : 1.f;

    // ---- argmax of the cleaned row (also the fallback of a degenerate row) ----
    ArgBest best{-INFINITY, 0x7fffffff};
    // 16 bytes a load, four loads in flight (a row of 152 thousand logits: 20 -> measured below us); a thread
    // sees its elements in rising order, so the first of equal values stays
    const int V4 = (((uintptr_t)l & 15) == 0) ? (V & ~3) : 0;
    for (int i0 = 4 * tid; i0 < V4; i0 += 16 * SMP_THREADS) {
        float4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 4 * SMP_THREADS;
            q[u] = i < V4 ? *reinterpret_cast<const float4*>(l + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 4 * SMP_THREADS;
            if (i < V4) {
                const float e[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float v = clean(e[j], 1.f);
                    if (best.i == 0x7fffffff || v > best.v) best = ArgBest{v, i + j};
                }
            }
        }
    }
    for (int i = V4 + tid; i < V; i += SMP_THREADS) {
        const float v = clean(l[i], 1.f);
        best = better(best, ArgBest{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) { s_f[warp] = best.v; s_i[warp] = best.i; }
    __syncthreads();
    if (tid == 0) {
        ArgBest b{s_f[0], s_i[0]};
        for (int w = 1; w < SMP_THREADS / 32; ++w) b = better(b, ArgBest{s_f[w], s_i[w]});
        s_pick = b.i == 0x7fffffff ? 0 : b.i;
        s_max = b.v * inv_t;
    }
    __syncthreads();
    const int arg = s_pick;
    const float row_max = s_max;               // maximum of the scaled row (top-k keeps it)
    const bool degenerate = !(row_max > -INFINITY && row_max < INFINITY);
    if (greedy && !out_logprob) {
        if (tid == 0) out_token[r] = arg;
        return;
    }

    // ---- top-k threshold by radix select on order-preserving keys ----
    unsigned kth_key = 0;                      // keep key >= kth_key
    if (!greedy && !degenerate && k > 0 && k < V) {
        if (tid == 0) { s_prefix = 0; s_remaining = (unsigned)k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_cnt[tid] = 0;
            __syncthreads();
            const unsigned prefix = s_prefix;
            const unsigned himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += SMP_THREADS) {
                const unsigned key = order_key(clean(l[i], inv_t));
                if ((key & himask) == prefix) atomicAdd(&s_cnt[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned rem = s_remaining, cum = 0;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + s_cnt[b] >= rem) break;
                    cum += s_cnt[b];
                }
                s_remaining = rem - cum;
                s_prefix = prefix | ((unsigned)b << shift);
            }
            __syncthreads();
        }
        kth_key = s_prefix;
    }

    // ---- total mass of the kept tokens (40-bit fixed point of exp(s - max)) ----
    unsigned long long mass = 0;
    if (!degenerate) {
        for (int i = tid; i < V; i += SMP_THREADS) {
            const float s = clean(l[i], inv_t);
            if (order_key(s) >= kth_key) mass += (unsigned long long)(expf(s - row_max) * SMP_FIX);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mass += __shfl_xor_sync(0xffffffffu, mass, o);
    if (lane == 0) s_w[warp] = mass;
    __syncthreads();
    if (tid == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < SMP_THREADS / 32; ++w) t += s_w[w];
        s_total = t;
    }
    __syncthreads();
    const unsigned long long total_k = s_total;   // mass after top-k

    if (greedy || degenerate || total_k == 0) {
        if (tid == 0) {
            out_token[r] = arg;
            if (out_logprob) {
                // log-softmax of the row at the argmax: exp(0) / sum
                out_logprob[r] = (degenerate || total_k == 0) ? 0.f : -logf((float)((double)total_k / (double)SMP_FIX));
            }
        }
        return;
    }

    // ---- nucleus threshold: radix select on keys weighted by mass ----
    unsigned nuc_key = kth_key;
    unsigned long long total = total_k;
    if (tp < 1.f) {
        const unsigned long long target = (unsigned long long)((double)tp * (double)total_k);
        if (tid == 0) { s_prefix = 0; s_above = 0; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_mass[tid] = 0;
            __syncthreads();
            const unsigned prefix = s_prefix;
            const unsigned himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += SMP_THREADS) {
                const float s = clean(l[i], inv_t);
                const unsigned key = order_key(s);
                if (key >= kth_key && (key & himask) == prefix) {
                    const unsigned long long q = (unsigned long long)(expf(s - row_max) * SMP_FIX);
                    if (q) atomicAdd(&s_mass[(key >> shift) & 255u], q);
                }
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long above = s_above;
                int b = 255;
                for (; b > 0; --b) {
                    if (above + s_mass[b] > target) break;   // crossing bin: cumulative exceeds top_p
                    above += s_mass[b];
                }
                s_above = above;
                s_prefix = prefix | ((unsigned)b << shift);
            }
            __syncthreads();
        }
        nuc_key = s_prefix > kth_key ? s_prefix : kth_key;
        // mass of the nucleus
        unsigned long long nm = 0;
        for (int i = tid; i < V; i += SMP_THREADS) {
            const float s = clean(l[i], inv_t);
            if (order_key(s) >= nuc_key) nm += (unsigned long long)(expf(s - row_max) * SMP_FIX);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) nm += __shfl_xor_sync(0xffffffffu, nm, o);
        __syncthreads();
        if (lane == 0) s_w[warp] = nm;
        __syncthreads();
        if (tid == 0) {
            unsigned long long t = 0;
            for (int w = 0; w < SMP_THREADS / 32; ++w) t += s_w[w];
            s_total = t;
        }
        __syncthreads();
        total = s_total;
    }

    // ---- inverse CDF in index order: warp w owns a contiguous span of the row ----
    const float u = uniform ? uniform[r] : 0.f;
    unsigned long long target = (unsigned long long)((double)u * (double)total);
    if (target >= total) target = total - 1;
    const int span = (V + 31) / 32;
    const int lo = warp * span, hi = min(V, lo + span);
    unsigned long long wsum = 0;
    for (int i = lo + lane; i < hi; i += 32) {
        const float s = clean(l[i], inv_t);
        if (order_key(s) >= nuc_key) wsum += (unsigned long long)(expf(s - row_max) * SMP_FIX);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
    __syncthreads();
    if (lane == 0) s_w[warp] = wsum;
    __syncthreads();
    unsigned long long before = 0;
    int owner = -1;
    for (int w = 0; w < 32; ++w) {
        if (owner < 0) {
            if (before + s_w[w] > target) owner = w; else before += s_w[w];
        }
    }
    if (owner < 0 && tid == 0) {
        out_token[r] = arg;
        if (out_logprob) out_logprob[r] = 0.f;
    }
    if (warp == owner) {
        unsigned long long run = before;
        int pick = -1;
        unsigned long long pick_q = 0;
        for (int base = lo; base < hi && pick < 0; base += 32) {
            const int i = base + lane;
            unsigned long long q = 0;
            if (i < hi) {
                const float s = clean(l[i], inv_t);
                if (order_key(s) >= nuc_key) q = (unsigned long long)(expf(s - row_max) * SMP_FIX);
            }
            unsigned long long inc = q;          // inclusive scan over the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long n = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += n;
            }
            const bool hit = q > 0 && run + inc > target;
            const unsigned ballot = __ballot_sync(0xffffffffu, hit);
            if (ballot) {
                const int first = __ffs(ballot) - 1;
                pick = base + first;
                pick_q = __shfl_sync(0xffffffffu, q, first);
            }
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) {
            out_token[r] = pick < 0 ? arg : pick;
            if (out_logprob)
                out_logprob[r] = pick < 0 ? 0.f : logf((float)((double)pick_q / (double)total));
        }
    }
}

extern "C" int vl_apply_penalties(float* logits, long long row_stride, int R, int V,
                                  const int* seen_off, const int* seen_ids,
                                  const float* repeat_p, const float* presence_p,
                                  const int* bias_off, const int* bias_ids, const float* bias_vals,
                                  void* stream) {
    if (R <= 0) return VL_OK;
    apply_penalties_kernel<<<R, 256, 0, (cudaStream_t)stream>>>(
        logits, row_stride, V, seen_off, seen_ids, repeat_p, presence_p, bias_off, bias_ids, bias_vals);
    return vl_launch_status();
}

extern "C" int vl_sample(const float* logits, long long row_stride, int R, int V,
                         const float* temperature, const int* top_k, const float* top_p,
                         const float* uniform, int* out_token, float* out_logprob, void* stream) {
    if (R <= 0) return VL_OK;
    if (V <= 0) return VL_ERR_ARGUMENT;
    return vl_launch(sample_kernel, dim3(R), dim3(SMP_THREADS), 0, (cudaStream_t)stream,
                     logits, row_stride, V, temperature, top_k, top_p, uniform, out_token, out_logprob);
}
