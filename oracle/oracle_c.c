/*
 * CPU oracle in plain C (TEST INFRASTRUCTURE ONLY; never linked into the product library).
 *
 * Same algorithm as oracle/oracle.py, written with loops so that full-size
 * workloads finish in seconds and so that the benchmark has a multi-threaded
 * CPU arm to time.  Reference lines followed (paths inside the reference project):
 *   encode           ucm/sparse/gsa_on_device/hash_encoder.py:359-370
 *   token distance   ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:148-182
 *   block min        ucm/sparse/gsa_on_device/hamming_topk.py:45-47,
 *                    ucm/sparse/gsa_on_device/csrc/cuda/hash_retrieval/cpy/hash_retrieval_backend.cpp:361-389
 *   top-k            hamming_topk.py:49-54 and hash_retrieval_backend.cpp:396-406, with the
 *                    (score, id) total order the reference leaves open
 *   seq_lens         hamming_topk.py:7-12
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC oracle_c.c -o _build/liboracle.so
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_MIN 0
#define ORC_SUM 1
#define ORC_SCORE_INVALID (-1)

int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the OpenMP team size (launchers such as torchrun export OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline float bf16_to_f32(uint16_t v)
{
    uint32_t u = ((uint32_t)v) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* codes_out[r, w] bit b = (sum_k x[r,k]*R[k,32w+b] > 0), float32 accumulation in k order. */
int orc_hash_encode(const uint16_t* x, int64_t rows, int64_t row_stride, const uint16_t* R,
                    int in_dim, int hash_bits, uint32_t* codes_out)
{
    if (hash_bits % 32 != 0 || in_dim <= 0) return -1;
    const int W = hash_bits / 32;
    float* Rf = (float*)malloc(sizeof(float) * (size_t)in_dim * hash_bits);
    if (!Rf) return -2;
    for (int64_t i = 0; i < (int64_t)in_dim * hash_bits; ++i) Rf[i] = bf16_to_f32(R[i]);
#pragma omp parallel
    {
        float* acc = (float*)malloc(sizeof(float) * hash_bits);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            for (int c = 0; c < hash_bits; ++c) acc[c] = 0.f;
            const uint16_t* xr = x + r * row_stride;
            for (int k = 0; k < in_dim; ++k) {
                const float xv = bf16_to_f32(xr[k]);
                const float* rr = Rf + (size_t)k * hash_bits;
                for (int c = 0; c < hash_bits; ++c) acc[c] += xv * rr[c];
            }
            for (int w = 0; w < W; ++w) {
                uint32_t word = 0;
                for (int b = 0; b < 32; ++b) word |= (uint32_t)(acc[32 * w + b] > 0.f) << b;
                codes_out[r * W + w] = word;
            }
        }
        free(acc);
    }
    free(Rf);
    return 0;
}

/* out [B, Hout, max_blocks] int32; ORC_SCORE_INVALID for blocks past the request's length. */
int orc_block_scores(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q,
                     int Hq, const int32_t* block_table, int max_blocks, const int32_t* seq_lens,
                     int B, int mode, int reduce_kvhead, int32_t* out)
{
    if (Hkv <= 0 || Hq % Hkv != 0) return -1;
    const int G = Hq / Hkv;
    const int Hout = reduce_kvhead ? 1 : Hkv;
    const int64_t total = (int64_t)B * max_blocks;
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t it = 0; it < total; ++it) {
        const int b = (int)(it / max_blocks), j = (int)(it % max_blocks);
        const int sl = seq_lens[b];
        const int nb = (sl + BS - 1) / BS;
        int32_t* o = out + (int64_t)b * Hout * max_blocks + j;
        if (j >= nb) {
            for (int h = 0; h < Hout; ++h) o[(int64_t)h * max_blocks] = ORC_SCORE_INVALID;
            continue;
        }
        const int64_t phys = block_table[(int64_t)b * max_blocks + j];
        if (phys < 0 || phys >= NB) {
#pragma omp atomic write
            bad = 1;
            continue;
        }
        const int ntok = (sl - j * BS) < BS ? (sl - j * BS) : BS;
        const uint32_t* blk = codes + phys * (int64_t)BS * Hkv * W;
        int64_t red = (mode == ORC_SUM) ? 0 : INT64_MAX;
        for (int h = 0; h < Hkv; ++h) {
            int64_t acc = (mode == ORC_SUM) ? 0 : INT64_MAX;
            for (int t = 0; t < ntok; ++t) {
                const uint32_t* kc = blk + ((int64_t)t * Hkv + h) * W;
                int d = 0;
                for (int g = 0; g < G; ++g) {
                    const uint32_t* qc = q + ((int64_t)b * Hq + h * G + g) * W;
                    for (int w = 0; w < W; ++w) d += __builtin_popcount(kc[w] ^ qc[w]);
                }
                if (mode == ORC_SUM) acc += d;
                else if (d < acc) acc = d;
            }
            if (reduce_kvhead) {
                if (mode == ORC_SUM) red += acc;
                else if (acc < red) red = acc;
            } else {
                o[(int64_t)h * max_blocks] = (int32_t)acc;
            }
        }
        if (reduce_kvhead) o[0] = (int32_t)red;
    }
    return bad ? -3 : 0;
}

typedef struct { uint32_t key; int32_t id; } orc_kv;

static int cmp_key_id(const void* a, const void* b)
{
    const orc_kv *x = (const orc_kv*)a, *y = (const orc_kv*)b;
    if (x->key != y->key) return x->key < y->key ? -1 : 1;
    return (x->id > y->id) - (x->id < y->id);
}
static int cmp_id(const void* a, const void* b)
{
    const orc_kv *x = (const orc_kv*)a, *y = (const orc_kv*)b;
    return (x->id > y->id) - (x->id < y->id);
}

static int is_forced(int j, int nb, int sl, int BS, const int32_t* must, int n_must, int sink,
                     int recent)
{
    if (j >= nb) return 0;
    for (int m = 0; m < n_must; ++m) {
        const int t = must[m] >= 0 ? must[m] : nb + must[m];
        if (t == j) return 1;
    }
    const int lo = j * BS;
    const int hi = (lo + BS < sl) ? lo + BS : sl;
    if (sink > 0 && lo < sink) return 1;
    if (recent > 0 && hi > sl - recent) return 1;
    return 0;
}

/*
 * scores [B,Hout,max_blocks] (from orc_block_scores) -> selections.
 * logical/physical/sel_scores [B,Hout,k]; valid_count/new_seq_lens [B].
 */
int orc_select(const int32_t* scores, int B, int Hout, int max_blocks, const int32_t* block_table,
               const int32_t* seq_lens, int BS, int k, const int32_t* k_per_request,
               const uint8_t* request_mask, const int32_t* must, int n_must, int sink, int recent,
               int32_t* logical, int32_t* physical, int32_t* sel_scores, int32_t* valid_count,
               int32_t* new_seq_lens)
{
    if (k > max_blocks || k < 0) return -1;
#pragma omp parallel
    {
        orc_kv* buf = (orc_kv*)malloc(sizeof(orc_kv) * (size_t)(max_blocks > 0 ? max_blocks : 1));
#pragma omp for schedule(dynamic, 1)
        for (int row = 0; row < B * Hout; ++row) {
            const int b = row / Hout;
            const int sl = seq_lens[b];
            const int nb = (sl + BS - 1) / BS;
            int kb = k;
            if (k_per_request) { kb = k_per_request[b]; if (kb < 0) kb = 0; if (kb > k) kb = k; }
            const int32_t* s = scores + (int64_t)row * max_blocks;
            int32_t* lo = logical + (int64_t)row * k;
            int32_t* po = physical + (int64_t)row * k;
            int32_t* so = sel_scores ? sel_scores + (int64_t)row * k : NULL;
            for (int i = 0; i < k; ++i) { lo[i] = -1; po[i] = 0; if (so) so[i] = -1; }
            const int masked = request_mask && !request_mask[b];
            if (masked) {
                for (int i = 0; i < kb; ++i) {
                    lo[i] = i; po[i] = block_table[(int64_t)b * max_blocks + i];
                    if (so) so[i] = s[i];
                }
            } else {
                for (int j = 0; j < max_blocks; ++j) {
                    uint32_t key;
                    if (s[j] == ORC_SCORE_INVALID) key = 0xFFFFFFFFu;
                    else if (is_forced(j, nb, sl, BS, must, n_must, sink, recent)) key = 0;
                    else key = (uint32_t)s[j] + 1u;
                    buf[j].key = key; buf[j].id = j;
                }
                qsort(buf, max_blocks, sizeof(orc_kv), cmp_key_id);
                qsort(buf, kb, sizeof(orc_kv), cmp_id);
                for (int i = 0; i < kb; ++i) {
                    lo[i] = buf[i].id;
                    po[i] = block_table[(int64_t)b * max_blocks + buf[i].id];
                    if (so) so[i] = s[buf[i].id];
                }
            }
            if (row % Hout == 0) {
                valid_count[b] = kb < nb ? kb : nb;
                int ns = sl;
                if (!masked) {
                    int over = sl - kb * BS; if (over < 0) over = 0;
                    ns = sl - ((over + BS - 1) / BS) * BS;
                }
                new_seq_lens[b] = ns;
            }
        }
        free(buf);
    }
    return 0;
}

/* out[b, i*BS+t, h, :] = pool[physical[b,(h),i], t, h, :]; row_bytes = D * elem size. */
int orc_gather_kv(const uint8_t* pool, int64_t NB, int BS, int Hkv, int64_t row_bytes,
                  const int32_t* physical, int B, int k, int per_head, uint8_t* out)
{
    const int64_t tok_bytes = (int64_t)Hkv * row_bytes, blk_bytes = tok_bytes * BS;
    int bad = 0;
#pragma omp parallel for schedule(static)
    for (int64_t it = 0; it < (int64_t)B * k; ++it) {
        const int b = (int)(it / k), i = (int)(it % k);
        uint8_t* dst = out + it * blk_bytes;
        if (!per_head) {
            const int64_t p = physical[(int64_t)b * k + i];
            if (p < 0 || p >= NB) { bad = 1; continue; }
            memcpy(dst, pool + p * blk_bytes, blk_bytes);
        } else {
            for (int h = 0; h < Hkv; ++h) {
                const int64_t p = physical[((int64_t)b * Hkv + h) * k + i];
                if (p < 0 || p >= NB) { bad = 1; continue; }
                for (int t = 0; t < BS; ++t)
                    memcpy(dst + t * tok_bytes + h * row_bytes,
                           pool + p * blk_bytes + t * tok_bytes + h * row_bytes, row_bytes);
            }
        }
    }
    return bad ? -3 : 0;
}
