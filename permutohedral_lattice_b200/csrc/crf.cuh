// The pointwise half of a dense-CRF mean-field update, fused into one pass over memory:
//   q_out = softmax over labels of ( -unaries - (wb * q_bilateral + ws * q_spatial) @ compatibility ).
// The two filtered label distributions come from the lattice filter (appearance and smoothness kernels);
// this kernel replaces the scale, add, matrix product, subtraction and softmax passes that would each
// read and write all points x labels floats.  The reference library ships no CRF code (its README names
// CRF-as-RNN as its user), so this follows the published mean-field update, not a reference file.
#pragma once
#include "common.cuh"

namespace pl {

// Row stride of the shared-memory tiles: odd, so that threads reading their own point's row never share a bank.
__host__ __device__ __forceinline__ int crf_row_stride(int L) { return L | 1; }

__host__ __forceinline__ size_t crf_smem_bytes(int tpb, int L) {
    return sizeof(float) * ((size_t)2 * tpb * crf_row_stride(L) + (size_t)L * L);
}

// One CTA per TPB consecutive points, whose [point][label] blocks are contiguous in memory: the block is
// loaded with coalesced accesses (message and negated unaries formed on the way), then one thread per
// point does the L x L product, the softmax, and the block leaves the same way it came.
// compat == nullptr: Potts model (1 - identity): pairwise_k = sum_j m_j - m_k.
// LT > 0: Potts model with the label count fixed at compile time (a point's rows then live in registers:
// one shared-memory read and one write per value); LT == 0: any count, any compatibility (rows stay in
// shared memory).
template <int TPB, int LT>
__global__ void __launch_bounds__(TPB)
crf_update(float* __restrict__ q_out, const float* __restrict__ unaries, const float* __restrict__ qb,
           const float* __restrict__ qs, const float* __restrict__ compat, float wb, float ws,
           long long n_points, int L) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int LS = crf_row_stride(L);
    float* m_s = reinterpret_cast<float*>(smem_raw);   // [TPB][LS] message, later the result
    float* z_s = m_s + (size_t)TPB * LS;               // [TPB][LS] -unaries, later the logits
    float* c_s = z_s + (size_t)TPB * LS;               // [L][L]
    const int tid = threadIdx.x;
    const long long p0 = (long long)blockIdx.x * TPB;
    const int np = (int)min((long long)TPB, n_points - p0);
    const int total = np * L;
    const size_t g0 = (size_t)p0 * L;
    if (compat)
        for (int i = tid; i < L * L; i += TPB) c_s[i] = compat[i];
    // element e = tid, tid + TPB, ... is label j of point p; (p, j) advance without a division
    const int DP = TPB / L, DJ = TPB % L;
    {
        int p = tid / L, j = tid - p * L;
        for (int e = tid; e < total; e += TPB) {
            m_s[p * LS + j] = PL_FADD(PL_FMUL(wb, qb[g0 + e]), PL_FMUL(ws, qs[g0 + e]));
            z_s[p * LS + j] = -unaries[g0 + e];
            p += DP;
            j += DJ;
            if (j >= L) {
                j -= L;
                p++;
            }
        }
    }
    __syncthreads();
    if (tid < np) {
        float* m = m_s + tid * LS;
        float* z = z_s + tid * LS;
        if constexpr (LT > 0) {
            float mr[LT], zr[LT];
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < LT; j++) {
                mr[j] = m[j];
                zr[j] = z[j];
                sum = PL_FADD(sum, mr[j]);
            }
            float mx = -INFINITY;
#pragma unroll
            for (int k = 0; k < LT; k++) {
                zr[k] = PL_FADD(zr[k], -PL_FADD(sum, -mr[k]));
                mx = fmaxf(mx, zr[k]);
            }
            float den = 0.f;
#pragma unroll
            for (int k = 0; k < LT; k++) {
                zr[k] = expf(PL_FADD(zr[k], -mx));
                den = PL_FADD(den, zr[k]);
            }
            const float inv = PL_FDIV(1.f, den);
#pragma unroll
            for (int k = 0; k < LT; k++) m[k] = PL_FMUL(zr[k], inv);
        } else {
            float mx = -INFINITY;
            if (compat) {
                for (int k = 0; k < L; k++) {
                    float pair = 0.f;
                    for (int j = 0; j < L; j++) pair = PL_FMA(m[j], c_s[j * L + k], pair);
                    const float zk = PL_FADD(z[k], -pair);
                    z[k] = zk;
                    mx = fmaxf(mx, zk);
                }
            } else {
                float sum = 0.f;
                for (int j = 0; j < L; j++) sum = PL_FADD(sum, m[j]);
                for (int k = 0; k < L; k++) {
                    const float zk = PL_FADD(z[k], -PL_FADD(sum, -m[k]));
                    z[k] = zk;
                    mx = fmaxf(mx, zk);
                }
            }
            float den = 0.f;
            for (int k = 0; k < L; k++) {
                const float ex = expf(PL_FADD(z[k], -mx));
                m[k] = ex;
                den = PL_FADD(den, ex);
            }
            const float inv = PL_FDIV(1.f, den);
            for (int k = 0; k < L; k++) m[k] = PL_FMUL(m[k], inv);
        }
    }
    __syncthreads();
    {
        int p = tid / L, j = tid - p * L;
        for (int e = tid; e < total; e += TPB) {
            q_out[g0 + e] = m_s[p * LS + j];
            p += DP;
            j += DJ;
            if (j >= L) {
                j -= L;
                p++;
            }
        }
    }
}

}  // namespace pl
