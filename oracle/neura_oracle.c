/*
 * CPU oracle for the quantized-linear path of Neura (test infrastructure only).
 *
 * This file is a plain-C restatement of the reference's host arithmetic for the
 * path "GGUF block pack/unpack -> linear layer product -> fused pointwise
 * epilogue".  It exists so that the CUDA library can be checked against it; no
 * product code calls into it.  Every function cites the reference file it
 * follows (paths are relative to the reference's repository root).
 *
 * Parity status: the block *layouts* are pinned (block byte counts from
 * crates/neura-abi/tests/layout.rs:148-158, the Q4_K walk by three independent
 * restatements inside the reference, and by the published GGML layout).  The
 * *quantiser* (which nibble/int8 code a float becomes) is "parity unpinned":
 * the reference holds no known-answer test for Q8_0, Q4_K or Q6_K bytes and cannot be
 * compiled here (no Rust toolchain), so the quantiser follows the reference's
 * source by reading only.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off: the reference's Rust
 * never contracts a*b+c into an fma, so neither may this file).
 */
#include <math.h>
#include <float.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define NRO_SINGLE 0u
#define NRO_HALF 1u
#define NRO_BFLOAT16 2u
#define NRO_Q8_0 8u /* crates/neura-abi/src/element.rs:3-17 (enum discriminants) */
#define NRO_Q4K 9u
#define NRO_Q5K 10u
#define NRO_Q6K 11u
#define NRO_Q3K 12u

#define QUANT_BLOCK 32      /* element.rs:35 */
#define SUPER_BLOCK 256     /* element.rs:36 */
#define SUPER_SUB_BLOCK 32  /* element.rs:37 */
#define SUPER_SCALE_BYTES 12 /* element.rs:40 */
#define Q8_0_BYTES 34       /* element.rs:155-158: 2 + 32 */
#define Q4K_BYTES 144       /* element.rs:159-162: 4 + 12 + 128 */
#define SUPER_SMALL_BLOCK 16 /* element.rs:38 */
#define Q6K_BYTES 210       /* element.rs:167-170: 2 + 128 + 64 + 16 */
#define Q5K_BYTES 176       /* element.rs:163-166: 4 + 12 + 32 + 128 */
#define Q3K_BYTES 110       /* element.rs:171-174: 32 + 64 + 12 + 2 */

/* ------------------------------------------------------------------ */
/* IEEE binary16 <-> binary32, round-to-nearest-even, subnormals kept. */
/* The reference calls crate `half` 2.7.1 (Cargo.lock:98-99) at        */
/* crates/neura-precision/src/ggml.rs:75,79,410; this restates the     */
/* published IEEE 754 conversion that crate implements.                */
/* ------------------------------------------------------------------ */
static uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

uint16_t nro_f32_to_f16(float value) {
    uint32_t x = f32_bits(value);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mag = x & 0x7fffffffu;
    if (mag >= 0x7f800000u) { /* inf / nan */
        if (mag > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((mag >> 13) & 0x3ffu));
        return (uint16_t)(sign | 0x7c00u);
    }
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf: >= 65520 */
    if (mag < 0x38800000u) { /* below 2^-14: subnormal half or zero */
        if (mag < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to zero */
        uint32_t exp = mag >> 23;
        uint32_t man = (mag & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126u - exp; /* 14..24 */
        uint32_t half = man >> shift;
        uint32_t rest = man & ((1u << shift) - 1u);
        uint32_t mid = 1u << (shift - 1u);
        if (rest > mid || (rest == mid && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((mag >> 13) - (112u << 10));
    uint32_t rest = mag & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

float nro_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        float v = (float)man * (1.0f / 16777216.0f); /* man * 2^-24, exact */
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* crates/neura-precision/src/lib.rs:325-329 */
uint16_t nro_bf16_rne(float value) {
    uint32_t bits = f32_bits(value);
    uint32_t rounded = bits + (0x7fffu + ((bits >> 16) & 1u));
    return (uint16_t)(rounded >> 16);
}

float nro_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* ------------------------------------------------------------------ */
/* PRNG: crates/neura-graph/src/init.rs:86-96                          */
/* ------------------------------------------------------------------ */
static float unit(uint32_t *entropy) {
    *entropy ^= *entropy << 13;
    *entropy ^= *entropy >> 17;
    *entropy ^= *entropy << 5;
    return (float)(*entropy >> 8) / (float)(1u << 24);
}

static float normal(uint32_t *entropy) {
    float u = unit(entropy);
    if (!(u > FLT_MIN)) u = FLT_MIN; /* f32::max(MIN_POSITIVE) */
    float radius = sqrtf(-2.0f * logf(u));
    return radius * cosf(6.28318530717958647692f * unit(entropy));
}

/* Init::Uniform{low,high}.samples (init.rs:63-70); the state is read and
 * written back so that consecutive tensors can share one stream. */
void nro_uniform(uint32_t *entropy, float low, float high, uint64_t count, float *out) {
    for (uint64_t i = 0; i < count; ++i) out[i] = low + (high - low) * unit(entropy);
}

/* Init::Normal{mean,deviation}.samples (init.rs:71-79) */
void nro_normal(uint32_t *entropy, float mean, float deviation, uint64_t count, float *out) {
    for (uint64_t i = 0; i < count; ++i) out[i] = mean + deviation * normal(entropy);
}

/* ------------------------------------------------------------------ */
/* Block geometry: crates/neura-abi/src/element.rs:145-178,231-268     */
/* ------------------------------------------------------------------ */
int nro_block(uint32_t element, uint32_t *elements, uint32_t *bytes) {
    switch (element) {
    case NRO_Q8_0: *elements = QUANT_BLOCK; *bytes = Q8_0_BYTES; return 0;
    case NRO_Q4K: *elements = SUPER_BLOCK; *bytes = Q4K_BYTES; return 0;
    case NRO_Q6K: *elements = SUPER_BLOCK; *bytes = Q6K_BYTES; return 0;
    case NRO_Q5K: *elements = SUPER_BLOCK; *bytes = Q5K_BYTES; return 0;
    case NRO_Q3K: *elements = SUPER_BLOCK; *bytes = Q3K_BYTES; return 0;
    case NRO_HALF: case NRO_BFLOAT16: *elements = 1; *bytes = 2; return 0;   /* element.rs:134: two to a word */
    default: return -1;
    }
}

uint64_t nro_payload_bytes(uint32_t element, uint64_t elements) {
    uint32_t per, bytes;
    if (element == NRO_SINGLE) return elements * 4u;
    if (nro_block(element, &per, &bytes)) return 0;
    return (elements + per - 1) / per * bytes;
}

/* payload rounded up to whole 4-byte words, as pack() pads it (ggml.rs:17-18) */
uint64_t nro_packed_bytes(uint32_t element, uint64_t elements) {
    return (nro_payload_bytes(element, elements) + 3u) / 4u * 4u;
}

/* ------------------------------------------------------------------ */
/* Host quantiser: crates/neura-precision/src/ggml.rs                  */
/* ------------------------------------------------------------------ */
static float least(float a, float b) { return a < b ? a : b; }       /* ggml.rs:90-92 */
static float greatest(float a, float b) { return a > b ? a : b; }    /* ggml.rs:94-96 */
static float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

static void put_half(uint8_t *field, int at, float value) { /* ggml.rs:78-80 */
    uint16_t h = nro_f32_to_f16(value);
    field[at] = (uint8_t)(h & 0xff);
    field[at + 1] = (uint8_t)(h >> 8);
}
static float half_at(const uint8_t *field, int at) { /* ggml.rs:74-76 */
    return nro_f16_to_f32((uint16_t)(field[at] | (field[at + 1] << 8)));
}

/* ggml.rs:201-209 (q8_0) with peak() from :98-108 */
static void q8_0_encode(const float *values, uint8_t *out) {
    float size = 0.0f;
    for (int i = 0; i < QUANT_BLOCK; ++i)
        if (size < fabsf(values[i])) size = fabsf(values[i]);
    float quantum = size / 127.0f;
    float inverse = quantum == 0.0f ? 0.0f : 1.0f / quantum;
    put_half(out, 0, quantum);
    for (int i = 0; i < QUANT_BLOCK; ++i) {
        float code = clampf(roundf(values[i] * inverse), -127.0f, 127.0f);
        out[2 + i] = (uint8_t)(int8_t)code;
    }
}

/* ggml.rs:211-216 */
static void q8_0_decode(const uint8_t *field, float *out) {
    float quantum = half_at(field, 0);
    for (int i = 0; i < QUANT_BLOCK; ++i) out[i] = (float)(int8_t)field[2 + i] * quantum;
}

/* ggml.rs:127-136 */
static void scale_min_k4(const uint8_t *scales, int at, uint32_t *scale, uint32_t *min) {
    if (at < 4) {
        *scale = scales[at] & 63u;
        *min = scales[at + 4] & 63u;
    } else {
        *scale = (uint32_t)(scales[at + 4] & 0x0f) | ((uint32_t)(scales[at - 4] >> 6) << 4);
        *min = (uint32_t)(scales[at + 4] >> 4) | ((uint32_t)(scales[at] >> 6) << 4);
    }
}

/* ggml.rs:138-147 */
static void put_scale_min_k4(uint8_t *scales, int at, uint32_t scale, uint32_t min) {
    if (at < 4) {
        scales[at] = (uint8_t)scale;
        scales[at + 4] = (uint8_t)min;
    } else {
        scales[at + 4] = (uint8_t)((scale & 0x0f) | ((min & 0x0f) << 4));
        scales[at - 4] |= (uint8_t)((scale >> 4) << 6);
        scales[at] |= (uint8_t)((min >> 4) << 6);
    }
}

static float scale_of(float quantum, float low) { return quantum == 0.0f ? 0.0f : low / quantum; } /* :116-118 */

static uint32_t quantized(float value, float quantum, float low, float high) { /* :120-125 */
    if (quantum == 0.0f) return 0;
    return (uint32_t)clampf(roundf(value / quantum), low, high);
}

/* affine_block (ggml.rs:149-199) with sub = 32: steps = 15 and the codes at byte 16 for q4_k (:314-316); steps = 31,
 * the low nibbles at byte 48 and the fifth bits at byte 16 for q5_k (:310-312) */
static void affine_encode(const float *values, uint8_t *field, int fifth) {
    const int count = SUPER_BLOCK / SUPER_SUB_BLOCK;
    const float steps = fifth ? 31.0f : 15.0f;
    const int quants = fifth ? 48 : 16;
    float lows[8], quantums[8];
    for (int at = 0; at < count; ++at) {
        float low = 0.0f, high = 0.0f; /* span(): fold from (0, 0) */
        for (int i = 0; i < SUPER_SUB_BLOCK; ++i) {
            float v = values[at * SUPER_SUB_BLOCK + i];
            low = least(low, v);
            high = greatest(high, v);
        }
        lows[at] = least(0.0f, low);
        quantums[at] = (high - lows[at]) / steps;
    }
    float scale = 0.0f, min = 0.0f;
    for (int at = 0; at < count; ++at) scale = greatest(scale, quantums[at]);
    scale = scale / 63.0f;
    for (int at = 0; at < count; ++at) min = greatest(min, -lows[at]);
    min = min / 63.0f;
    uint8_t codes[8], mins[8];
    for (int at = 0; at < count; ++at) {
        codes[at] = (uint8_t)clampf(roundf(scale_of(scale, quantums[at])), 0.0f, 63.0f);
        mins[at] = (uint8_t)clampf(roundf(scale_of(min, -lows[at])), 0.0f, 63.0f);
    }
    uint8_t scales[SUPER_SCALE_BYTES];
    memset(scales, 0, sizeof scales);
    for (int at = 0; at < count; ++at) put_scale_min_k4(scales, at, codes[at], mins[at]);
    memset(field, 0, fifth ? Q5K_BYTES : Q4K_BYTES);
    put_half(field, 0, scale);
    put_half(field, 2, min);
    memcpy(field + 4, scales, SUPER_SCALE_BYTES);
    for (int at = 0; at < count; ++at) {
        /* the codes are taken with the unrounded f32 scale and min, not the stored halves */
        float quantum = scale * (float)codes[at];
        float low = min * (float)mins[at];
        for (int within = 0; within < SUPER_SUB_BLOCK; ++within) {
            uint32_t code = quantized(values[at * SUPER_SUB_BLOCK + within] + low, quantum, 0.0f, steps);
            int group = at / 2;
            int seat = at % 2;
            field[quants + group * SUPER_SUB_BLOCK + within] |= (uint8_t)((code & 0x0f) << (seat ? 4 : 0));
            if (fifth && (code & 0x10u)) field[16 + within] |= (uint8_t)(1u << (2 * group + seat));
        }
    }
}

static void q4_k_encode(const float *values, uint8_t *field) { affine_encode(values, field, 0); }
static void q5_k_encode(const float *values, uint8_t *field) { affine_encode(values, field, 1); }

/* ggml.rs:336-350 */
static void q4_k_decode(const uint8_t *field, float *out) {
    float scale = half_at(field, 0);
    float min = half_at(field, 2);
    int n = 0;
    for (int group = 0; group < 4; ++group) {
        for (int seat = 0; seat < 2; ++seat) {
            uint32_t code, offset;
            scale_min_k4(field + 4, group * 2 + seat, &code, &offset);
            float quantum = scale * (float)code;
            float low = min * (float)offset;
            for (int within = 0; within < SUPER_SUB_BLOCK; ++within) {
                uint8_t byte = field[16 + group * 32 + within];
                uint32_t quant = seat ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 0x0f);
                out[n++] = quantum * (float)quant - low;
            }
        }
    }
}

/* q5_k_values (ggml.rs:318-334): q4_k's walk with a fifth bit per code, bit 2 group + seat of byte 16 + within */
static void q5_k_decode(const uint8_t *field, float *out) {
    float scale = half_at(field, 0);
    float min = half_at(field, 2);
    int n = 0;
    for (int group = 0; group < 4; ++group) {
        for (int seat = 0; seat < 2; ++seat) {
            uint32_t code, offset;
            scale_min_k4(field + 4, group * 2 + seat, &code, &offset);
            float quantum = scale * (float)code;
            float low = min * (float)offset;
            for (int within = 0; within < SUPER_SUB_BLOCK; ++within) {
                uint8_t byte = field[48 + group * 32 + within];
                uint32_t high = (uint32_t)(field[16 + within] >> (2 * group + seat)) & 1u;
                uint32_t quant = (seat ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 0x0f)) | (high << 4);
                out[n++] = quantum * (float)quant - low;
            }
        }
    }
}

/* q3_k_scale / put_q3_k_scale (ggml.rs:222-241): sixteen six-bit codes; the low nibbles of codes 0-7 and 8-15 share
 * bytes 0-7, the top two bits of codes at, at + 4, at + 8, at + 12 share byte 8 + at % 4 */
static uint32_t q3_k_scale(const uint8_t *scales, int at) {
    uint8_t low = scales[at % 8];
    uint32_t nibble = at < 8 ? (uint32_t)(low & 0x0f) : (uint32_t)(low >> 4);
    return nibble | ((((uint32_t)scales[8 + at % 4] >> (2 * (at / 4))) & 3u) << 4);
}
static void put_q3_k_scale(uint8_t *scales, int at, uint32_t code) {
    if (at < 8) scales[at] |= (uint8_t)(code & 0x0f);
    else scales[at - 8] |= (uint8_t)((code & 0x0f) << 4);
    scales[8 + at % 4] |= (uint8_t)(((code >> 4) & 3u) << (2 * (at / 4)));
}

/* Where number `at` of a q3_k block keeps its two low bits (byte, shift) and its third bit (byte, bit)
 * (ggml.rs:267-281, :292-300): runs of 16, eight runs a half; run `within` of a half sits in bit pair within / 2 of
 * byte half * 32 + (within % 2) * 16 + lane */
static void q3_k_seat(int at, int *byte, int *shift, int *mask_byte, int *mask_bit) {
    int sub = at / 16, lane = at % 16, half = sub / 8, within = sub % 8, j = within / 2, second = within % 2;
    *byte = 32 + half * 32 + second * 16 + lane;
    *shift = 2 * j;
    *mask_byte = second * 16 + lane;
    *mask_bit = half * 4 + j;
}

/* q3_k (ggml.rs:243-290): one d for the block, a six-bit scale (biased by 32) for every run of 16, codes -4..3 */
static void q3_k_encode(const float *values, uint8_t *field) {
    float peaks[16], widest = 0.0f;
    for (int at = 0; at < 16; ++at) {
        peaks[at] = 0.0f;
        for (int i = 0; i < 16; ++i) peaks[at] = greatest(peaks[at], fabsf(values[at * 16 + i]));
        widest = greatest(widest, peaks[at]);
    }
    if (!(widest > FLT_MIN)) widest = FLT_MIN;   /* .max(f32::MIN_POSITIVE) */
    float d = widest / 4.0f / 31.0f;
    uint32_t codes[16];
    memset(field, 0, Q3K_BYTES);
    for (int at = 0; at < 16; ++at) {
        codes[at] = (uint32_t)clampf(roundf(peaks[at] / 4.0f / d), 0.0f, 31.0f) + 32u;
        put_q3_k_scale(field + 96, at, codes[at]);
    }
    for (int at = 0; at < SUPER_BLOCK; ++at) {
        float quantum = d * (float)(codes[at / 16] - 32u);
        int quant = quantum == 0.0f ? 0 : (int)clampf(roundf(values[at] / quantum), -4.0f, 3.0f);
        int byte, shift, mask_byte, mask_bit;
        q3_k_seat(at, &byte, &shift, &mask_byte, &mask_bit);
        field[byte] |= (uint8_t)(((uint32_t)quant & 3u) << shift);
        if (quant >= 0) field[mask_byte] |= (uint8_t)(1u << mask_bit);
    }
    put_half(field, 108, d);
}

/* q3_k_values (ggml.rs:292-308) */
static void q3_k_decode(const uint8_t *field, float *out) {
    float d = half_at(field, 108);
    for (int at = 0; at < SUPER_BLOCK; ++at) {
        int byte, shift, mask_byte, mask_bit;
        q3_k_seat(at, &byte, &shift, &mask_byte, &mask_bit);
        int low = (field[byte] >> shift) & 3;
        int quant = low - ((field[mask_byte] >> mask_bit) & 1 ? 0 : 4);
        out[at] = d * ((float)(uint8_t)q3_k_scale(field + 96, at / 16) - 32.0f) * (float)quant;
    }
}

/* peak (ggml.rs:98-108): the largest magnitude of a run (the first to reach it wins) */
static float peak_size(const float *values, int count) {
    float size = 0.0f;
    for (int i = 0; i < count; ++i)
        if (size < fabsf(values[i])) size = fabsf(values[i]);
    return size;
}

/* `(value / quantum).round().clamp(low, high) as u32` (ggml.rs:120-125) for a range that reaches below zero: Rust's
 * float-to-unsigned cast saturates, so every negative quotient becomes 0.  (q6_k calls it with low = -32: a negative
 * weight packs as code 0 + 32, which decodes as zero.  This file follows the reference, not the GGML quantiser.) */
static uint32_t quantized_saturating(float value, float quantum, float low, float high) {
    if (quantum == 0.0f) return 0;
    float r = clampf(roundf(value / quantum), low, high);
    return r <= 0.0f ? 0u : (uint32_t)r;
}

/* q6_k (ggml.rs:352-393): sixteen runs of 16 with an int8 scale each, six-bit codes biased by 32 */
static void q6_k_encode(const float *values, uint8_t *field) {
    const int sub = SUPER_SMALL_BLOCK, count = SUPER_BLOCK / SUPER_SMALL_BLOCK;
    float factors[16];
    for (int at = 0; at < count; ++at) factors[at] = peak_size(values + at * sub, sub) / 32.0f;
    float scale = 0.0f;
    for (int at = 0; at < count; ++at) scale = greatest(scale, fabsf(factors[at]));
    scale = scale / 127.0f;
    memset(field, 0, Q6K_BYTES);
    put_half(field, 208, scale);
    for (int at = 0; at < count; ++at) {
        int8_t code = 0;
        if (scale != 0.0f) code = (int8_t)clampf(roundf(factors[at] / scale), -127.0f, 127.0f);
        field[192 + at] = (uint8_t)code;
        float factor = scale * (float)code;
        for (int within = 0; within < sub; ++within) {
            int element = at * sub + within;
            int half = element / 128, group = (element % 128) / 32, seat = element % 32;
            uint32_t quant = quantized_saturating(values[element], factor, -32.0f, 31.0f) + 32u;
            field[half * 64 + (group % 2) * 32 + seat] |= (uint8_t)((quant & 0x0fu) << (group >= 2 ? 4 : 0));
            field[128 + half * 32 + seat] |= (uint8_t)(((quant >> 4) & 3u) << (2 * group));
        }
    }
}

/* q6_k_values (ggml.rs:395-407) */
static void q6_k_decode(const uint8_t *field, float *out) {
    float scale = half_at(field, 208);
    int at = 0;
    for (int seat = 0; seat < 2; ++seat)
        for (int group = 0; group < 4; ++group)
            for (int within = 0; within < SUPER_SUB_BLOCK; ++within) {
                int index = group * 2 + within / 16;
                int8_t sub = (int8_t)field[192 + seat * 8 + index];
                uint8_t packed = field[seat * 64 + (group % 2) * 32 + within];
                uint32_t quant = (group >= 2 ? packed >> 4 : packed & 0x0fu) | (((field[128 + seat * 32 + within] >> (2 * group)) & 3u) << 4);
                out[at++] = scale * (float)sub * ((float)quant - 32.0f);
            }
}

/* pack(): ggml.rs:8-20.  `out` must hold nro_packed_bytes(element, count). */
int nro_pack(uint32_t element, const float *values, uint64_t count, uint8_t *out) {
    uint32_t per, bytes;
    if (nro_block(element, &per, &bytes)) return -1;
    uint64_t blocks = (count + per - 1) / per;
    if (element == NRO_HALF || element == NRO_BFLOAT16) { /* crates/neura-precision/src/lib.rs:8-9: two to a word, the first low */
        for (uint64_t i = 0; i < count; ++i) {
            uint16_t h = element == NRO_HALF ? nro_f32_to_f16(values[i]) : nro_bf16_rne(values[i]);
            out[2 * i] = (uint8_t)(h & 0xff);
            out[2 * i + 1] = (uint8_t)(h >> 8);
        }
        blocks = count;
    }
    else for (uint64_t b = 0; b < blocks; ++b) {
        float held[SUPER_BLOCK];
        memset(held, 0, sizeof held);
        uint64_t have = count - b * per < per ? count - b * per : per;
        memcpy(held, values + b * per, have * sizeof(float));
        if (element == NRO_Q8_0) q8_0_encode(held, out + b * bytes);
        else if (element == NRO_Q6K) q6_k_encode(held, out + b * bytes);
        else if (element == NRO_Q5K) q5_k_encode(held, out + b * bytes);
        else if (element == NRO_Q3K) q3_k_encode(held, out + b * bytes);
        else q4_k_encode(held, out + b * bytes);
    }
    uint64_t end = blocks * bytes;
    uint64_t padded = (end + 3u) / 4u * 4u;
    for (uint64_t i = end; i < padded; ++i) out[i] = 0;
    return 0;
}

/* unpack(): ggml.rs:22-38 */
int nro_unpack(uint32_t element, uint64_t count, const uint8_t *bytes_in, float *out) {
    uint32_t per, bytes;
    if (nro_block(element, &per, &bytes)) return -1;
    uint64_t blocks = (count + per - 1) / per;
    if (element == NRO_HALF || element == NRO_BFLOAT16) { /* crates/neura-precision/src/lib.rs:34-42 */
        for (uint64_t i = 0; i < count; ++i) {
            uint16_t h = (uint16_t)(bytes_in[2 * i] | (bytes_in[2 * i + 1] << 8));
            out[i] = element == NRO_HALF ? nro_f16_to_f32(h) : nro_bf16_to_f32(h);
        }
        return 0;
    }
    for (uint64_t b = 0; b < blocks; ++b) {
        float held[SUPER_BLOCK];
        if (element == NRO_Q8_0) q8_0_decode(bytes_in + b * bytes, held);
        else if (element == NRO_Q6K) q6_k_decode(bytes_in + b * bytes, held);
        else if (element == NRO_Q5K) q5_k_decode(bytes_in + b * bytes, held);
        else if (element == NRO_Q3K) q3_k_decode(bytes_in + b * bytes, held);
        else q4_k_decode(bytes_in + b * bytes, held);
        uint64_t have = count - b * per < per ? count - b * per : per;
        memcpy(out + b * per, held, have * sizeof(float));
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* Second restatement of the decoders, after the device code's scalar  */
/* fetch: crates/neura-kernel/src/fetch.rs:183-267.  Used by the tests */
/* to cross-pin the walk above (the reference states it three times).  */
/* ------------------------------------------------------------------ */
static uint32_t ggml_byte(const uint8_t *heap, uint64_t at) { return heap[at]; }

static uint32_t ggml_k4_scale(const uint8_t *heap, uint64_t base, uint32_t at) { /* fetch.rs:209-218 */
    int upper = at >= 4u;
    uint32_t seat = upper ? at - 4u : 0u;
    uint32_t low = upper ? (ggml_byte(heap, base + at + 4u) & 0xfu) : (ggml_byte(heap, base + at) & 63u);
    return low | (upper ? ((ggml_byte(heap, base + seat) >> 6) << 4) : 0u);
}

static uint32_t ggml_k4_min(const uint8_t *heap, uint64_t base, uint32_t at) { /* fetch.rs:220-225 */
    int upper = at >= 4u;
    uint32_t packed = ggml_byte(heap, base + at + 4u);
    uint32_t low = upper ? packed >> 4 : packed & 63u;
    return low | (upper ? ((ggml_byte(heap, base + at) >> 6) << 4) : 0u);
}

float nro_fetch(uint32_t element, const uint8_t *heap, uint64_t at) {
    if (element == NRO_Q8_0) { /* fetch.rs:236-240 */
        uint64_t base = at / QUANT_BLOCK * Q8_0_BYTES;
        uint32_t byte = ggml_byte(heap, base + 2u + at % QUANT_BLOCK);
        float signed_code = (float)((int32_t)byte - (byte >= 128u ? 256 : 0));
        return signed_code * half_at(heap + base, 0);
    }
    if (element == NRO_Q4K) { /* fetch.rs:256-267 */
        uint64_t base = at / SUPER_BLOCK * Q4K_BYTES;
        uint32_t within = (uint32_t)(at % SUPER_BLOCK);
        uint32_t group = within / 64u;
        uint32_t seat = (within % 64u) / SUPER_SUB_BLOCK;
        uint32_t lane = within % SUPER_SUB_BLOCK;
        uint32_t sub = group * 2u + seat;
        uint32_t packed = ggml_byte(heap, base + 16u + group * 32u + lane);
        uint32_t quant = seat == 1u ? packed >> 4 : packed & 0xfu;
        float a = half_at(heap + base, 0) * (float)ggml_k4_scale(heap, base + 4u, sub);
        float b = half_at(heap + base, 2) * (float)ggml_k4_min(heap, base + 4u, sub);
        return a * (float)quant - b;
    }
    if (element == NRO_HALF || element == NRO_BFLOAT16) { /* fetch.rs:95-107 */
        uint16_t h = (uint16_t)(heap[2 * at] | (heap[2 * at + 1] << 8));
        return element == NRO_HALF ? nro_f16_to_f32(h) : nro_bf16_to_f32(h);
    }
    if (element == NRO_Q5K) { /* fetch.rs:269-282 */
        uint64_t base = at / SUPER_BLOCK * Q5K_BYTES;
        uint32_t within = (uint32_t)(at % SUPER_BLOCK);
        uint32_t group = within / 64u, seat = (within % 64u) / SUPER_SUB_BLOCK, lane = within % SUPER_SUB_BLOCK;
        uint32_t sub = group * 2u + seat;
        uint32_t packed = ggml_byte(heap, base + 48u + group * 32u + lane);
        uint32_t nibble = seat == 1u ? packed >> 4 : packed & 0xfu;
        uint32_t fifth = (ggml_byte(heap, base + 16u + lane) >> (2u * group + seat)) & 1u;
        float a = half_at(heap + base, 0) * (float)ggml_k4_scale(heap, base + 4u, sub);
        float b = half_at(heap + base, 2) * (float)ggml_k4_min(heap, base + 4u, sub);
        return a * (float)(nibble | (fifth << 4)) - b;
    }
    if (element == NRO_Q3K) { /* fetch.rs:226-233 (ggml_q3_scale), :242-254 */
        uint64_t base = at / SUPER_BLOCK * Q3K_BYTES;
        uint32_t within = (uint32_t)(at % SUPER_BLOCK);
        uint32_t half = within / 128u, local = within % 128u, j = local / 32u, seat = local % 32u;
        uint32_t index = half * 8u + j * 2u + seat / 16u;
        uint32_t low_byte = ggml_byte(heap, base + 96u + index % 8u);
        uint32_t nibble = index >= 8u ? low_byte >> 4 : low_byte & 0x0fu;
        uint32_t code = nibble | (((ggml_byte(heap, base + 96u + 8u + index % 4u) >> (2u * (index / 4u))) & 3u) << 4);
        float scale = (float)code - 32.0f;
        uint32_t low = (ggml_byte(heap, base + 32u + half * 32u + seat) >> (2u * j)) & 3u;
        uint32_t high = (ggml_byte(heap, base + seat) >> (half * 4u + j)) & 1u;
        float quant = (float)low - (high == 0u ? 4.0f : 0.0f);
        return half_at(heap + base, 108) * scale * quant;
    }
    if (element == NRO_Q6K) { /* fetch.rs:284-301 */
        uint64_t base = at / SUPER_BLOCK * Q6K_BYTES;
        uint32_t within = (uint32_t)(at % SUPER_BLOCK);
        uint32_t half = within / 128u, seat = within % 128u;
        uint32_t group = seat / SUPER_SUB_BLOCK, lane = seat % SUPER_SUB_BLOCK;
        uint32_t packed = ggml_byte(heap, base + half * 64u + (group % 2u) * 32u + lane);
        uint32_t low = group >= 2u ? packed >> 4 : packed & 0xfu;
        uint32_t high = (ggml_byte(heap, base + 128u + half * 32u + lane) >> (2u * group)) & 3u;
        uint32_t quant = low | (high << 4);
        uint32_t scale = ggml_byte(heap, base + 192u + half * 8u + group * 2u + lane / 16u);
        float signed_scale = (float)((int32_t)scale - (scale >= 128u ? 256 : 0));
        return half_at(heap + base, 208) * signed_scale * ((float)quant - 32.0f);
    }
    return NAN;
}

/* ------------------------------------------------------------------ */
/* Pointwise epilogue: crates/neura-pointwise/src/op.rs:141-170 (op    */
/* codes in declaration order) and neura-kernel/src/pointwise.rs:66-68 */
/* ------------------------------------------------------------------ */
enum {
    OP_ADD = 0, OP_MUL, OP_SUB, OP_DIV, OP_MAXIMUM, OP_MINIMUM, OP_RELU, OP_SQRT, OP_RECIP, OP_EXP,
    OP_LOG, OP_TANH, OP_SIGMOID, OP_NEG, OP_ABS, OP_IDENTITY, OP_SIN, OP_COS, OP_POW, OP_FLOOR,
    OP_GELU, OP_SILU
};

static float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

float nro_op_apply(uint32_t op, float a, float b) {
    switch (op) {
    case OP_ADD: return a + b;
    case OP_MUL: return a * b;
    case OP_SUB: return a - b;
    case OP_DIV: return a / b;
    case OP_MAXIMUM: return a > b ? a : b;
    case OP_MINIMUM: return a < b ? a : b;
    case OP_RELU: return a > 0.0f ? a : 0.0f;
    case OP_SQRT: return sqrtf(a);
    case OP_RECIP: return 1.0f / a;
    case OP_EXP: return expf(a);
    case OP_LOG: return logf(a);
    case OP_TANH: return tanhf(a);
    case OP_SIGMOID: return sigmoidf(a);
    case OP_NEG: return -a;
    case OP_ABS: return fabsf(a);
    case OP_IDENTITY: return a;
    case OP_SIN: return sinf(a);
    case OP_COS: return cosf(a);
    case OP_POW: return powf(a, b);
    case OP_FLOOR: return floorf(a);
    case OP_GELU: {
        float inner = 0.7978845608f * (a + 0.044715f * a * a * a);
        return 0.5f * a * (1.0f + tanhf(inner));
    }
    case OP_SILU: return a * sigmoidf(a);
    default: return NAN;
    }
}

/* One step of `chained` (pointwise.rs:90-104): operand is fetched at the output
 * coordinate through broadcast strides; `swapped` puts the operand first. */
typedef struct {
    uint32_t op;
    uint32_t swapped;
    const float *operand;   /* NULL: the step is unary (operand reads as 0) */
    int64_t row_stride;     /* elements between output rows of the operand (0 = broadcast) */
    int64_t col_stride;     /* elements between output columns of the operand (0 = broadcast) */
} nro_step;

static float chained(const nro_step *steps, uint32_t n_steps, uint64_t row, uint64_t col, float carried) {
    float result = carried;
    for (uint32_t s = 0; s < n_steps; ++s) {
        float operand = steps[s].operand
            ? steps[s].operand[(int64_t)row * steps[s].row_stride + (int64_t)col * steps[s].col_stride]
            : 0.0f;
        result = steps[s].swapped ? nro_op_apply(steps[s].op, operand, result)
                                  : nro_op_apply(steps[s].op, result, operand);
    }
    return result;
}

/* ------------------------------------------------------------------ */
/* The product itself.  The reference has no host matmul; its tests    */
/* state the expected result as a sequential f32 loop over             */
/* unpack(pack(w)) (crates/neura-runtime/tests/runtime.rs:72-83):      */
/*   total += weight[column*depth + step] * inputs[row*depth + step]   */
/* ------------------------------------------------------------------ */
typedef struct {
    uint32_t element;
    const uint8_t *packed; /* N rows, each ceil(K/per) blocks, row-major, K contiguous */
    const float *weight;   /* or: already unpacked f32 [N][K] (packed == NULL) */
    const float *x;        /* [rows][x_stride] */
    float *out;            /* [rows][out_stride] */
    uint64_t rows, n, k, x_stride, out_stride;
    const nro_step *steps;
    uint32_t n_steps;
    uint64_t c0, c1;       /* column range of this worker */
    int round_bf16;        /* prefill variant: weights and activations rounded to bf16 first */
} product_job;

static void *product_worker(void *arg) {
    product_job *job = (product_job *)arg;
    uint32_t per = 1, bytes = 4;
    if (job->packed) nro_block(job->element, &per, &bytes);
    uint64_t row_bytes = (job->k + per - 1) / per * bytes;
    float *held = (float *)malloc(((job->k + per - 1) / per * per) * sizeof(float));
    for (uint64_t c = job->c0; c < job->c1; ++c) {
        const float *w;
        if (job->packed) {
            nro_unpack(job->element, job->k, job->packed + c * row_bytes, held);
            w = held;
        } else {
            w = job->weight + c * job->k;
        }
        if (job->round_bf16) {
            if (w != held) memcpy(held, w, job->k * sizeof(float));
            for (uint64_t s = 0; s < job->k; ++s) held[s] = nro_bf16_to_f32(nro_bf16_rne(held[s]));
            w = held;
        }
        for (uint64_t r = 0; r < job->rows; ++r) {
            const float *x = job->x + r * job->x_stride;
            float total = 0.0f;
            if (job->round_bf16) {
                for (uint64_t s = 0; s < job->k; ++s) total += w[s] * nro_bf16_to_f32(nro_bf16_rne(x[s]));
            } else {
                for (uint64_t s = 0; s < job->k; ++s) total += w[s] * x[s];
            }
            job->out[r * job->out_stride + c] = chained(job->steps, job->n_steps, r, c, total);
        }
    }
    free(held);
    return NULL;
}

static int run_product(product_job base, int threads) {
    if (threads < 1) threads = 1;
    if ((uint64_t)threads > base.n) threads = (int)(base.n ? base.n : 1);
    pthread_t *ids = (pthread_t *)malloc(sizeof(pthread_t) * threads);
    product_job *jobs = (product_job *)malloc(sizeof(product_job) * threads);
    for (int t = 0; t < threads; ++t) {
        jobs[t] = base;
        jobs[t].c0 = base.n * t / threads;
        jobs[t].c1 = base.n * (t + 1) / threads;
        if (threads == 1) product_worker(&jobs[t]);
        else pthread_create(&ids[t], NULL, product_worker, &jobs[t]);
    }
    if (threads > 1)
        for (int t = 0; t < threads; ++t) pthread_join(ids[t], NULL);
    free(ids);
    free(jobs);
    return 0;
}

/* out[r][c] = chain(sum_k unpack(W)[c][k] * x[r][k]); rows of W are packed
 * independently (each row is a whole number of blocks, as a GGUF stores it). */
int nro_linear(uint32_t element, const uint8_t *packed, uint64_t n, uint64_t k, const float *x, uint64_t rows,
               uint64_t x_stride, float *out, uint64_t out_stride, const nro_step *steps, uint32_t n_steps,
               int threads) {
    uint32_t per, bytes;
    if (nro_block(element, &per, &bytes) || k % per) return -1;
    product_job job = {element, packed, NULL, x, out, rows, n, k, x_stride, out_stride, steps, n_steps, 0, 0, 0};
    return run_product(job, threads);
}

/* Prefill variant: dequantised weights and the activations are rounded to
 * bf16 (RNE) before the f32 product, which is what the tensor-core path does. */
int nro_linear_bf16(uint32_t element, const uint8_t *packed, uint64_t n, uint64_t k, const float *x,
                    uint64_t rows, uint64_t x_stride, float *out, uint64_t out_stride, const nro_step *steps,
                    uint32_t n_steps, int threads) {
    uint32_t per, bytes;
    if (nro_block(element, &per, &bytes) || k % per) return -1;
    product_job job = {element, packed, NULL, x, out, rows, n, k, x_stride, out_stride, steps, n_steps, 0, 0, 1};
    return run_product(job, threads);
}

/* The reference tests' loop on an already unpacked weight (runtime.rs:72-83). */
int nro_matmul_f32(const float *weight, uint64_t n, uint64_t k, const float *x, uint64_t rows, float *out,
                   int threads) {
    product_job job = {NRO_SINGLE, NULL, weight, x, out, rows, n, k, k, n, NULL, 0, 0, 0, 0};
    return run_product(job, threads);
}

/* ------------------------------------------------------------------ */
/* The steps either side of the products in a decoder layer.          */
/* ------------------------------------------------------------------ */

/* rms_norm: crates/neura-kernel/src/task/norm.rs:55-131 with op = NORM_RMS:
 * scale = 1 / sqrt(mean(x^2) + floor); out = x * scale * weight.
 * (composed form in crates/neura-runtime/tests/norm.rs:21-26) */
void nro_rms_norm(const float *x, const float *weight, float floor, uint64_t rows, uint64_t width, float *out) {
    for (uint64_t r = 0; r < rows; ++r) {
        const float *row = x + r * width;
        float square = 0.0f;
        for (uint64_t c = 0; c < width; ++c) square = square + row[c] * row[c];
        float scale = 1.0f / sqrtf(square / (float)width + floor);
        for (uint64_t c = 0; c < width; ++c) {
            float result = row[c] * scale;
            if (weight) result = result * weight[c];
            out[r * width + c] = result;
        }
    }
}

/* rope: crates/neura-kernel/src/task/rope.rs:48-122 (half rotation), CPU form in
 * crates/neura-runtime/tests/runtime.rs:468-494.  x is [rows][heads][width]; every head of
 * row r turns by position[r]. */
void nro_rope(float *x, const uint32_t *position, float base, uint64_t rows, uint64_t heads, uint64_t width) {
    uint64_t half = width / 2;
    for (uint64_t r = 0; r < rows; ++r) {
        for (uint64_t h = 0; h < heads; ++h) {
            float *v = x + (r * heads + h) * width;
            for (uint64_t c = 0; c < half; ++c) {
                float angle = (float)position[r] * powf(base, -2.0f * (float)c / (float)width);
                float cosine = cosf(angle), sine = sinf(angle);
                float low = v[c], high = v[c + half];
                v[c] = low * cosine - high * sine;
                v[c + half] = high * cosine + low * sine;
            }
        }
    }
}

/* Causal grouped-query attention of one new row per sequence over its cache:
 * crates/neura-runtime/tests/support/attention.rs:71-109 (softmax(q.k * scale) v, query head h
 * reads key head h / (heads / key_heads), attention.rs:19-27), in f32 like the device
 * (crates/neura-kernel/src/task/attention.rs:309-617).
 *   q      [batch][heads][width]
 *   keys   [batch][key_heads][capacity][width]   (positions 0..count[b]-1 are live)
 *   out    [batch][heads][width] */
void nro_attend(const float *q, const float *keys, const float *values, const uint32_t *count, float scale,
                uint64_t batch, uint64_t heads, uint64_t key_heads, uint64_t capacity, uint64_t width, float *out) {
    uint64_t group = heads / key_heads;
    float *logits = (float *)malloc(capacity * sizeof(float));
    for (uint64_t b = 0; b < batch; ++b) {
        for (uint64_t h = 0; h < heads; ++h) {
            const float *query = q + (b * heads + h) * width;
            const float *k = keys + ((b * key_heads + h / group) * capacity) * width;
            const float *v = values + ((b * key_heads + h / group) * capacity) * width;
            float largest = -INFINITY;
            for (uint64_t p = 0; p < count[b]; ++p) {
                float total = 0.0f;
                for (uint64_t d = 0; d < width; ++d) total = total + query[d] * k[p * width + d];
                logits[p] = total * scale;
                if (logits[p] > largest) largest = logits[p];
            }
            float total = 0.0f;
            for (uint64_t p = 0; p < count[b]; ++p) {
                logits[p] = expf(logits[p] - largest);
                total = total + logits[p];
            }
            for (uint64_t d = 0; d < width; ++d) {
                float sum = 0.0f;
                for (uint64_t p = 0; p < count[b]; ++p) sum = sum + logits[p] * v[p * width + d];
                out[(b * heads + h) * width + d] = sum / total;
            }
        }
    }
    free(logits);
}

/* argmax with the lowest index winning a tie: choice_precedes,
 * crates/neura-kernel/src/task/choice.rs:46-52 */
void nro_argmax(const float *x, uint64_t rows, uint64_t width, uint32_t *out) {
    for (uint64_t r = 0; r < rows; ++r) {
        uint32_t best = 0;
        for (uint64_t c = 1; c < width; ++c)
            if (x[r * width + c] > x[r * width + best]) best = (uint32_t)c;
        out[r] = best;
    }
}

/* gather of a quantised table row: run_gather (crates/neura-kernel/src/task/select.rs:29-49)
 * over fetch (fetch.rs) = the dequantised row. */
int nro_embed(uint32_t element, const uint8_t *packed, uint64_t width, const uint32_t *tokens, uint64_t rows,
              float *out) {
    uint32_t per, bytes;
    if (nro_block(element, &per, &bytes) || width % per) return -1;
    uint64_t row_bytes = width / per * bytes;
    for (uint64_t r = 0; r < rows; ++r)
        nro_unpack(element, width, packed + (uint64_t)tokens[r] * row_bytes, out + r * width);
    return 0;
}
