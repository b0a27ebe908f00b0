/* CPU restatement of the reference's Parakeet TDT decoder + joint: TEST INFRASTRUCTURE ONLY.
 *
 * Follows rust/parakeet-decoder/src/lib.rs loop for loop (that crate is what ships as
 * src/engines/asr-parakeet/parakeet-decoder.wasm):
 *   :49-68   expf / floorf / ldexpf / tanhf / sigmoid  (the crate's own approximations, f32)
 *   :117-130 dotv        four f32 lane accumulators, horizontal sum lane 0+1+2+3, scalar tail
 *   :133-147 lstm_step   ONNX iofc gate order, candidate state NH/NC
 *   :150-156 predict / commit_state
 *   :159-175 compute_predproj   axpy over the 640 outputs, k outer
 *   :179-227 joint_tail  relu(enc+pred), axpy over 8198 logits, rows with J[n]==0 skipped,
 *                        int8 out matrix: sc = J[n]*scale[n] first, then OUT += sc*(f32)q
 *   :236-254 joint       1024->640 projection, frame entries equal to 0 skipped
 *   :258-319 decode / decode_proj   greedy TDT loop, durations 0..4, MAX_SYMBOLS 10
 * Every multiply and add is rounded separately (wasm simd128 has no fused multiply-add): compile
 * with -ffp-contract=off.  Lane-parallel loops of the original give the same result as the scalar
 * loops here because their lanes never interact.
 *
 * Pinning: tests compare this file bit for bit (token ids, emission frames, and the logits of single
 * joint steps through tdt_joint_logits) with the shipped module executed by oracle/wasm_exec.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define EXPORT __attribute__((visibility("default")))

enum { HID = 640, ENC_D = 1024, VOCAB = 8193, LOGITS = 8198, BLANK = VOCAB - 1, MAX_SYMBOLS = 10 };

typedef struct {
    const float *embed, *lw[2], *lr[2], *lb[2], *enc_w, *enc_b, *pred_w, *pred_b, *out_w, *out_b;
    const int8_t *out_wq;
    const float *out_scale;
    float J[HID], OUT[LOGITS], ENCPROJ[HID], PREDPROJ[HID];
    float H[2][HID], C[2][HID], NH[2][HID], NC[2][HID], DECOUT[HID];
} tdt_t;

static inline float tdt_floorf(float x) {
    float i = (float)(int32_t)x;
    return i > x ? i - 1.0f : i;
}
static inline float tdt_ldexpf(float x, int32_t e) {
    float r = x;
    int32_t n = e;
    while (n > 30) { r *= 1073741824.0f; n -= 30; }
    while (n < -30) { r *= 9.313225746154785e-10f; n += 30; }
    uint32_t bits = ((uint32_t)(127 + n)) << 23;
    float p;
    memcpy(&p, &bits, 4);
    return r * p;
}
static inline float tdt_expf(float x) {
    float xc = x > 30.0f ? 30.0f : (x < -30.0f ? -30.0f : x);
    float t = xc * 1.4426950408889634f;
    float fl = tdt_floorf(t);
    float frac = t - fl;
    float p = 1.0f + frac * (0.6931472f + frac * (0.2402265f + frac * (0.0555041f + frac * 0.0096181f)));
    return tdt_ldexpf(p, (int32_t)fl);
}
static inline float tdt_sigmoid(float x) { return 1.0f / (1.0f + tdt_expf(-x)); }
static inline float tdt_tanhf(float x) {
    float e = tdt_expf(2.0f * x);
    return (e - 1.0f) / (e + 1.0f);
}

static float dotv(const float *a, const float *b, size_t n) {
    size_t n4 = n & ~(size_t)3;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    size_t i = 0;
    for (; i < n4; i += 4)
        for (int l = 0; l < 4; l++) {
            float p = a[i + l] * b[i + l];
            acc[l] = acc[l] + p;
        }
    float s = acc[0] + acc[1];
    s = s + acc[2];
    s = s + acc[3];
    for (; i < n; i++) {
        float p = a[i] * b[i];
        s += p;
    }
    return s;
}

static void lstm_step(tdt_t *d, int layer, const float *x) {
    const float *w = d->lw[layer], *r = d->lr[layer], *b = d->lb[layer];
    const float *hp = d->H[layer], *c = d->C[layer];
    for (size_t g = 0; g < HID; g++) {
        size_t wi = g * HID, wo = (HID + g) * HID, wf = (2 * HID + g) * HID, wc = (3 * HID + g) * HID;
        float zi = b[g] + b[4 * HID + g];
        zi = zi + dotv(w + wi, x, HID);
        zi = zi + dotv(r + wi, hp, HID);
        float zo = b[HID + g] + b[5 * HID + g];
        zo = zo + dotv(w + wo, x, HID);
        zo = zo + dotv(r + wo, hp, HID);
        float zf = b[2 * HID + g] + b[6 * HID + g];
        zf = zf + dotv(w + wf, x, HID);
        zf = zf + dotv(r + wf, hp, HID);
        float zc = b[3 * HID + g] + b[7 * HID + g];
        zc = zc + dotv(w + wc, x, HID);
        zc = zc + dotv(r + wc, hp, HID);
        float t1 = tdt_sigmoid(zf) * c[g];
        float t2 = tdt_sigmoid(zi) * tdt_tanhf(zc);
        float cc = t1 + t2;
        d->NC[layer][g] = cc;
        d->NH[layer][g] = tdt_sigmoid(zo) * tdt_tanhf(cc);
    }
}

static void predict(tdt_t *d, size_t token) {
    lstm_step(d, 0, d->embed + token * HID);
    lstm_step(d, 1, d->NH[0]);
    memcpy(d->DECOUT, d->NH[1], sizeof d->DECOUT);
}
static void commit_state(tdt_t *d) {
    memcpy(d->H, d->NH, sizeof d->H);
    memcpy(d->C, d->NC, sizeof d->C);
}
static void compute_predproj(tdt_t *d) {
    for (size_t n = 0; n < HID; n++) d->PREDPROJ[n] = d->pred_b[n];
    for (size_t k = 0; k < HID; k++) {
        float dk = d->DECOUT[k];
        const float *row = d->pred_w + k * HID;
        for (size_t n = 0; n < HID; n++) {
            float p = dk * row[n];
            d->PREDPROJ[n] = d->PREDPROJ[n] + p;
        }
    }
}

static void joint_tail(tdt_t *d) {
    for (size_t n = 0; n < HID; n++) {
        float v = d->ENCPROJ[n] + d->PREDPROJ[n];
        d->J[n] = v > 0.0f ? v : 0.0f;
    }
    for (size_t m = 0; m < LOGITS; m++) d->OUT[m] = d->out_b[m];
    if (d->out_wq) {
        for (size_t n = 0; n < HID; n++) {
            float jn = d->J[n];
            if (jn == 0.0f) continue;
            float sc = jn * d->out_scale[n];
            const int8_t *row = d->out_wq + n * LOGITS;
            for (size_t m = 0; m < LOGITS; m++) {
                float p = sc * (float)row[m];
                d->OUT[m] = d->OUT[m] + p;
            }
        }
        return;
    }
    for (size_t n = 0; n < HID; n++) {
        float jn = d->J[n];
        if (jn == 0.0f) continue;
        const float *row = d->out_w + n * LOGITS;
        for (size_t m = 0; m < LOGITS; m++) {
            float p = jn * row[m];
            d->OUT[m] = d->OUT[m] + p;
        }
    }
}
static void joint_pre(tdt_t *d, const float *proj) {
    memcpy(d->ENCPROJ, proj, sizeof d->ENCPROJ);
    joint_tail(d);
}
static void joint(tdt_t *d, const float *frame) {
    for (size_t n = 0; n < HID; n++) d->ENCPROJ[n] = d->enc_b[n];
    for (size_t k = 0; k < ENC_D; k++) {
        float fk = frame[k];
        if (fk == 0.0f) continue;
        const float *row = d->enc_w + k * HID;
        for (size_t n = 0; n < HID; n++) {
            float p = fk * row[n];
            d->ENCPROJ[n] = d->ENCPROJ[n] + p;
        }
    }
    joint_tail(d);
}

static int32_t decode_any(tdt_t *d, const float *frames, uint32_t tenc_, int32_t *out_ids, int32_t *out_frames, int pre) {
    memset(d->H, 0, sizeof d->H);
    memset(d->C, 0, sizeof d->C);
    size_t tenc = tenc_;
    int32_t n_out = 0;
    size_t last_tok = BLANK;
    predict(d, last_tok);
    compute_predproj(d);
    size_t t = 0;
    int32_t emitted = 0;
    while (t < tenc) {
        if (pre) joint_pre(d, frames + t * HID);
        else joint(d, frames + t * ENC_D);
        size_t max_id = 0;
        float max_v = -INFINITY;
        for (size_t i = 0; i < VOCAB; i++)
            if (d->OUT[i] > max_v) { max_v = d->OUT[i]; max_id = i; }
        size_t step = 0;
        float dv = -INFINITY;
        for (size_t i = VOCAB; i < LOGITS; i++)
            if (d->OUT[i] > dv) { dv = d->OUT[i]; step = i - VOCAB; }
        if (max_id != BLANK) {
            commit_state(d);
            last_tok = max_id;
            out_ids[n_out] = (int32_t)max_id;
            out_frames[n_out] = (int32_t)t;
            n_out += 1;
            emitted += 1;
            predict(d, last_tok);
            compute_predproj(d);
        }
        if (step > 0) { t += step; emitted = 0; }
        else if (max_id == BLANK || emitted >= MAX_SYMBOLS) { t += 1; emitted = 0; }
    }
    return n_out;
}

/* ---- C entry points (ctypes) ------------------------------------------------------------------ */

EXPORT void *tdt_create(const float *embed, const float *l0w, const float *l0r, const float *l0b, const float *l1w,
                        const float *l1r, const float *l1b, const float *enc_w, const float *enc_b,
                        const float *pred_w, const float *pred_b, const float *out_w, const float *out_b) {
    tdt_t *d = (tdt_t *)calloc(1, sizeof(tdt_t));
    if (!d) return NULL;
    d->embed = embed;
    d->lw[0] = l0w; d->lr[0] = l0r; d->lb[0] = l0b;
    d->lw[1] = l1w; d->lr[1] = l1r; d->lb[1] = l1b;
    d->enc_w = enc_w; d->enc_b = enc_b; d->pred_w = pred_w; d->pred_b = pred_b;
    d->out_w = out_w; d->out_b = out_b;
    return d;
}
EXPORT void tdt_set_out_q(void *h, const int8_t *q, const float *scale) {
    tdt_t *d = (tdt_t *)h;
    d->out_wq = q;
    d->out_scale = scale;
}
EXPORT void tdt_destroy(void *h) { free(h); }
EXPORT int32_t tdt_decode(void *h, const float *frames, uint32_t tenc, int32_t *ids, int32_t *fr) {
    return decode_any((tdt_t *)h, frames, tenc, ids, fr, 0);
}
EXPORT int32_t tdt_decode_proj(void *h, const float *proj, uint32_t tenc, int32_t *ids, int32_t *fr) {
    return decode_any((tdt_t *)h, proj, tenc, ids, fr, 1);
}
/* One joint step from zero state after predict(token): logits [8198] for a pre-projected frame. */
EXPORT void tdt_joint_logits(void *h, int32_t token, const float *proj, float *logits) {
    tdt_t *d = (tdt_t *)h;
    memset(d->H, 0, sizeof d->H);
    memset(d->C, 0, sizeof d->C);
    predict(d, (size_t)token);
    compute_predproj(d);
    joint_pre(d, proj);
    memcpy(logits, d->OUT, sizeof d->OUT);
}
/* Logits of the most recent joint step (the state a decode call leaves behind). */
EXPORT void tdt_last_logits(void *h, float *logits) { memcpy(logits, ((tdt_t *)h)->OUT, sizeof(float) * LOGITS); }
/* Many windows at once: window w reads proj + w*tenc*640, writes ids/fr + w*cap, counts[w]. */
EXPORT void tdt_decode_proj_batch(void *const *hs, int nthreads, const float *proj, uint32_t tenc, int32_t nwin,
                                  int32_t cap, int32_t *ids, int32_t *fr, int32_t *counts) {
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
    for (int32_t w = 0; w < nwin; w++) {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        counts[w] = decode_any((tdt_t *)hs[tid], proj + (size_t)w * tenc * HID, tenc, ids + (size_t)w * cap,
                               fr + (size_t)w * cap, 1);
    }
}
