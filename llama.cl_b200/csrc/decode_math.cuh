// Arithmetic shared by the decode FC kernels (rows <= 8): the in-kernel Q8 activation quantizer and the
// per-block integer dot product + fp32 scaling.  One copy, so that the kernels cannot drift apart in the
// parts that decide bit-exactness.
//
// Reference: FC_dynamic_quantize_x (ops/op_fc.hpp:246-268) with get_amax / quant_row_q8_0
// (ops/utils.hpp:177-220), and the inner loops of fc_Q4A (ops/op_fc.hpp:337-412).
#pragma once
#include "common.cuh"

namespace q4fc {

constexpr uint32_t kNibMask = 0x0F0F0F0Fu;

// D(16x8, s32) += A(16x32, u8) * B(32x8, s8).  A pure function of its operands: left to the scheduler.
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One warp quantizes 128 consecutive k of ROWS rows: lane l holds v[m][0..3] = x[m][k0 + 4l .. 4l+3].
// A K group spans SEG = G/4 lanes.  `len` = valid values of this lane's group (0: the group does not exist),
// `body` = len rounded down to 8 (the reference's vector body rounds half to even, its scalar tail half away
// from zero).  Out per row: the 4 codes packed little-endian, the scale d = amax/127 (IEEE division), and
// `aux` = the tree-ordered sum of the group's raw values, or with SIGNED the bits of 8 * (sum of codes).
// The reference's 1/16 activation scale of Q4_0 and its x16 nibble shift cancel exactly; neither is applied.
// The rows may have different `len` (q8_quantize_rows_v: rows that are different 128-k chunks of one activation row).
template <int G, int ROWS, bool SIGNED>
__device__ __forceinline__ void q8_quantize_rows_v(const float (&v)[ROWS][4], int lane, const int (&lens)[ROWS],
                                                   uint32_t (&packed)[ROWS], float (&d)[ROWS], float (&aux)[ROWS]) {
    constexpr int SEG = G / 4;
    const int e0 = (lane % SEG) * 4;
    float amax[ROWS], fsum[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; m++) {
        amax[m] = 0.0f, fsum[m] = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (e0 + j < lens[m]) {
                amax[m] = fmaxf(amax[m], fabsf(v[m][j]));
                fsum[m] += v[m][j];
            }
    }
    // the rows go through the same straight-line code so that their shuffle / divide chains overlap
#pragma unroll
    for (int off = SEG / 2; off > 0; off >>= 1) {
#pragma unroll
        for (int m = 0; m < ROWS; m++) {
            amax[m] = fmaxf(amax[m], __shfl_xor_sync(0xffffffffu, amax[m], off));
            fsum[m] += __shfl_xor_sync(0xffffffffu, fsum[m], off);
        }
    }
#pragma unroll
    for (int m = 0; m < ROWS; m++) {
        d[m] = div_const_rn(amax[m], 127.0f, 1.0f / 127.0f);
        const float id = inv_or_zero(d[m]);
        uint32_t pk = 0;
        int isum = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int q = 0;
            if (e0 + j < lens[m]) {
                const float tq = __fmul_rn(v[m][j], id);
                if (e0 + j < (lens[m] & ~7)) {
                    q = __float2int_rn(tq);  // nearest even
                } else {
                    const float h = __int_as_float((__float_as_int(tq) & 0x80000000) | 0x3F000000);
                    q = __float2int_rz(__fadd_rz(tq, h));  // half away from zero, exact for every fp32
                }
                q = min(127, max(-128, q));
            }
            isum += q;
            pk |= (uint32_t)(q & 0xFF) << (8 * j);
        }
        if (SIGNED) {
#pragma unroll
            for (int off = SEG / 2; off > 0; off >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, off);
        }
        packed[m] = pk;
        aux[m] = SIGNED ? __int_as_float(8 * isum) : fsum[m];
    }
}

template <int G, int ROWS, bool SIGNED>
__device__ __forceinline__ void q8_quantize_rows(const float (&v)[ROWS][4], int lane, int len, uint32_t (&packed)[ROWS],
                                                 float (&d)[ROWS], float (&aux)[ROWS]) {
    int lens[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; m++) lens[m] = len;
    q8_quantize_rows_v<G, ROWS, SIGNED>(v, lane, lens, packed, d, aux);
}

// One block (32 columns x G k) against <= 8 activation rows, for lane (g = lane >> 2, t = lane & 3):
//   q[j]   the lane's 128 bits of set j (block rows 4j + t, columns 4g..4g+3: byte offset (4j+t)*128 + 16g)
//   wd/wm  fp16 scales / minima of columns 4g..4g+3
//   codes  this lane's activation row g at the block's first k, plus 8t: 8 codes per set at +32j
//   sc     the block's 16 floats: (scale, aux) of rows 0..7
// The weight columns sit on the 16-row side of the MMA, the activation rows on its 8-column side; the k order
// is permuted the same way on both operands.  acc[c][mi] belongs to column 4g+c, row 2t+mi.
//
// Group 128 (four sets): the low nibbles of two sets fill one MMA (w & 0x0F0F0F0F), the high nibbles of the
// same two sets another one, left in place (w & 0xF0F0F0F0 = 16 x nibble, still a u8), so a word costs two
// logic operations instead of three; the two exact integer sums meet in fp32: I = IL + IH / 16, exact because
// IH is a multiple of 16 and everything stays below 2^24.  The integer ALU is the scarce pipe of this kernel;
// the conversions (XU pipe) and the extra FMA are free by comparison.
// Group 32 (one set): low nibbles in the first half of the MMA's k, shifted high nibbles in the second.
// MI = 1 (a launch with one activation row): only row 2t of the lane's two rows is converted and scaled; acc[c][1]
// is left as it is.
template <int G, int QTYPE, bool SIGNED, int MI = 2>
__device__ __forceinline__ void block_accumulate(const uint4 (&q)[G / 32], uint2 wd, uint2 wm, const uint8_t* codes,
                                                 bool row_live, const float* sc, int t, float (&acc)[4][2]) {
    constexpr int SETS = G / 32;
    float fI[4][2];
    const float4 s4 = *reinterpret_cast<const float4*>(sc + t * 4);  // scale, aux of rows 2t and 2t+1
    const float xs[2] = {s4.x, s4.z};
    const float gs[2] = {s4.y, s4.w};
    if constexpr (SETS == 4) {
        constexpr uint32_t kHiMask = 0xF0F0F0F0u;
        int il0[4] = {0, 0, 0, 0}, il1[4] = {0, 0, 0, 0}, ih0[4] = {0, 0, 0, 0}, ih1[4] = {0, 0, 0, 0};
#pragma unroll
        for (int pr = 0; pr < 2; pr++) {
            const uint4 qa = q[2 * pr], qb = q[2 * pr + 1];
            uint2 xa = make_uint2(0u, 0u), xb = make_uint2(0u, 0u);
            if (row_live) {
                xa = *reinterpret_cast<const uint2*>(codes + 64 * pr);
                xb = *reinterpret_cast<const uint2*>(codes + 64 * pr + 32);
            }
            uint32_t la0 = qa.x & kNibMask, la1 = qa.y & kNibMask, la2 = qa.z & kNibMask, la3 = qa.w & kNibMask;
            uint32_t lb0 = qb.x & kNibMask, lb1 = qb.y & kNibMask, lb2 = qb.z & kNibMask, lb3 = qb.w & kNibMask;
            uint32_t ha0 = qa.x & kHiMask, ha1 = qa.y & kHiMask, ha2 = qa.z & kHiMask, ha3 = qa.w & kHiMask;
            uint32_t hb0 = qb.x & kHiMask, hb1 = qb.y & kHiMask, hb2 = qb.z & kHiMask, hb3 = qb.w & kHiMask;
            if (SIGNED) {
                la0 ^= 0x08080808u, la1 ^= 0x08080808u, la2 ^= 0x08080808u, la3 ^= 0x08080808u;
                lb0 ^= 0x08080808u, lb1 ^= 0x08080808u, lb2 ^= 0x08080808u, lb3 ^= 0x08080808u;
                ha0 ^= 0x80808080u, ha1 ^= 0x80808080u, ha2 ^= 0x80808080u, ha3 ^= 0x80808080u;
                hb0 ^= 0x80808080u, hb1 ^= 0x80808080u, hb2 ^= 0x80808080u, hb3 ^= 0x80808080u;
            }
            mma_u8s8(il0, la0, la1, lb0, lb1, xa.x, xb.x);
            mma_u8s8(il1, la2, la3, lb2, lb3, xa.x, xb.x);
            mma_u8s8(ih0, ha0, ha1, hb0, hb1, xa.y, xb.y);
            mma_u8s8(ih1, ha2, ha3, hb2, hb3, xa.y, xb.y);
        }
        const int il[4][2] = {{il0[0], il0[1]}, {il0[2], il0[3]}, {il1[0], il1[1]}, {il1[2], il1[3]}};
        const int ih[4][2] = {{ih0[0], ih0[1]}, {ih0[2], ih0[3]}, {ih1[0], ih1[1]}, {ih1[2], ih1[3]}};
#pragma unroll
        for (int c = 0; c < 4; c++) {
#pragma unroll
            for (int mi = 0; mi < MI; mi++) {
                int L = il[c][mi];
                if (SIGNED) L -= __float_as_int(gs[mi]);
                // |IL|, |IH|/16 <= 15 * 127 * 64 and their sum < 2^24: every step is exact
                fI[c][mi] = fmaf(__int2float_rn(ih[c][mi]), 0.0625f, __int2float_rn(L));
            }
        }
    } else {
        int ia[4] = {0, 0, 0, 0}, ib[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < SETS; j++) {
            uint2 xb = make_uint2(0u, 0u);
            if (row_live) xb = *reinterpret_cast<const uint2*>(codes + 32 * j);
            uint32_t l0 = q[j].x & kNibMask, l1 = q[j].y & kNibMask, l2 = q[j].z & kNibMask, l3 = q[j].w & kNibMask;
            uint32_t h0 = (q[j].x >> 4) & kNibMask, h1 = (q[j].y >> 4) & kNibMask, h2 = (q[j].z >> 4) & kNibMask,
                     h3 = (q[j].w >> 4) & kNibMask;
            if (SIGNED) {
                l0 ^= 0x08080808u, l1 ^= 0x08080808u, l2 ^= 0x08080808u, l3 ^= 0x08080808u;
                h0 ^= 0x08080808u, h1 ^= 0x08080808u, h2 ^= 0x08080808u, h3 ^= 0x08080808u;
            }
            mma_u8s8(ia, l0, l1, h0, h1, xb.x, xb.y);
            mma_u8s8(ib, l2, l3, h2, h3, xb.x, xb.y);
        }
        const int iv[4][2] = {{ia[0], ia[1]}, {ia[2], ia[3]}, {ib[0], ib[1]}, {ib[2], ib[3]}};
#pragma unroll
        for (int c = 0; c < 4; c++) {
#pragma unroll
            for (int mi = 0; mi < MI; mi++) {
                int I = iv[c][mi];
                if (SIGNED) I -= __float_as_int(gs[mi]);
                fI[c][mi] = __int2float_rn(I);  // |I| <= 15 * 127 * 32: exact
            }
        }
    }
    const float2 wd01 = __half22float2(*reinterpret_cast<const __half2*>(&wd.x));
    const float2 wd23 = __half22float2(*reinterpret_cast<const __half2*>(&wd.y));
    const float wdf[4] = {wd01.x, wd01.y, wd23.x, wd23.y};
    float wmf[4] = {0.f, 0.f, 0.f, 0.f};
    if (QTYPE == 1) {
        const float2 wm01 = __half22float2(*reinterpret_cast<const __half2*>(&wm.x));
        const float2 wm23 = __half22float2(*reinterpret_cast<const __half2*>(&wm.y));
        wmf[0] = wm01.x, wmf[1] = wm01.y, wmf[2] = wm23.x, wmf[3] = wm23.y;
    }
#pragma unroll
    for (int c = 0; c < 4; c++) {
#pragma unroll
        for (int mi = 0; mi < MI; mi++) {
            acc[c][mi] = fmaf(__fmul_rn(wdf[c], xs[mi]), fI[c][mi], acc[c][mi]);
            if (QTYPE == 1) acc[c][mi] = fmaf(wmf[c], gs[mi], acc[c][mi]);
        }
    }
}

}  // namespace q4fc
