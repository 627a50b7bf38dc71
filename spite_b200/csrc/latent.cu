// Attention through latents: what happens between the products.
//
//  * latent_prepare: one row of the first product's float32 output holds a token's query latent, its
//    key/value latent, the key part that all heads share and the gate columns.  Both latents are RMS-normed
//    with a gain (float32 sums and scaling), the shared key part is rotated (neighbouring pairs, angle
//    position * inv_freq[i], cos and sin times an amplitude), and the cache row of the token's position
//    becomes [normed key/value latent ; rotated shared part ; zeros].  The gates become sigmoid(column).
//  * latent_queries: the rotating tail of every query head is rotated the same way into the row that the
//    attention kernels read ([kv_rank elements left for the product with the heads' key matrices ; rotated
//    tail ; zeros]), the (token, head) rows are listed head by head for the products per head, and the unrotated
//    parts are laid out in that order, so that the product that follows reads its rows in place.
//
// One block a token; float32 arithmetic whatever the element type.
#include "attention.cuh"

struct LatentPrepareParams {
    const float* down;          // [tokens, down_stride]: query latent, key/value latent, shared key part, gate columns
    long long down_stride;
    void* cq_out;               // [tokens, q_rank] normed query latent (activation type)
    const float* q_gain;        // [q_rank]
    const float* kv_gain;       // [kv_rank]
    const float* inv_freq;      // [rot_dim / 2]
    float rot_amplitude;
    float eps;
    int q_rank, kv_rank, rot_dim;
    int num_gates;
    float* gates_out;           // [tokens, num_gates] or null
    int write_cache;
};

struct LatentQueryParams {
    const void* q;              // [tokens, num_heads * (head_dim + rot_dim)]
    void* q_out;                // [tokens, num_heads * row]
    const float* inv_freq;      // [rot_dim / 2]
    float rot_amplitude;
    int num_heads, head_dim, rot_dim, kv_rank, row;
    const int* positions;       // [tokens]
    int n_tokens;
    int* rows_out;              // [num_heads * tokens]: rows_out[h * tokens + t] = t * num_heads + h
    int* offsets_out;           // [num_heads + 1]: offsets_out[h] = h * tokens
    void* q_sorted_out;         // [num_heads * tokens, head_dim] or null: the unrotated parts head by head (row h * tokens + t),
                                // the order in which the product with the heads' key matrices takes its rows
};

namespace {

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const LatentPrepareParams p, const StepTokens b,
                                                             const PagedCache c) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float* in = p.down + (size_t)t * p.down_stride;
    const int pos = b.positions[t];

    // query latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) { const float v = in[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    float mul = 1.0f / sqrtf(ss / (float)p.q_rank + p.eps);
    T* cq = (T*)p.cq_out + (size_t)t * p.q_rank;
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) cq[i] = from_f32<T>(in[i] * mul * p.q_gain[i]);

    // gates
    if (p.gates_out)
        for (int h = threadIdx.x; h < p.num_gates; h += blockDim.x)
            p.gates_out[(size_t)t * p.num_gates + h] = 1.0f / (1.0f + expf(-in[p.q_rank + p.kv_rank + p.rot_dim + h]));

    // key/value latent and the shared key part: the cache row of this position
    const float* kv = in + p.q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) { const float v = kv[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    if (!p.write_cache) return;
    const int page = b.block_table[(size_t)b.seg_of_token[t] * b.table_width + pos / c.page_size];
    if (page < 0 || page >= c.n_pages) return;               // the host never lets this happen
    mul = 1.0f / sqrtf(ss / (float)p.kv_rank + p.eps);
    T* row = (T*)c.kv + ((size_t)page * c.page_size + pos % c.page_size) * c.head_dim;
    for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) row[i] = from_f32<T>(kv[i] * mul * p.kv_gain[i]);
    const float* kr = kv + p.kv_rank;
    for (int i = threadIdx.x; 2 * i < p.rot_dim; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
        sn *= p.rot_amplitude; cs *= p.rot_amplitude;
        const float a = kr[2 * i], bb = kr[2 * i + 1];
        row[p.kv_rank + 2 * i] = from_f32<T>(a * cs - bb * sn);
        row[p.kv_rank + 2 * i + 1] = from_f32<T>(bb * cs + a * sn);
    }
    for (int i = p.kv_rank + p.rot_dim + threadIdx.x; i < c.head_dim; i += blockDim.x) row[i] = from_f32<T>(0.f);
}

template <typename T>
__global__ void __launch_bounds__(128) latent_queries_kernel(const LatentQueryParams p) {
    extern __shared__ float cs_sn[];                         // [rot_dim / 2] cos, then as many sin
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int half = p.rot_dim / 2;
    const int pos = p.positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
        cs_sn[i] = cs * p.rot_amplitude;
        cs_sn[half + i] = sn * p.rot_amplitude;
    }
    __syncthreads();
    const int qh = p.head_dim + p.rot_dim;
    const T* q = (const T*)p.q + (size_t)t * p.num_heads * qh;
    T* out = (T*)p.q_out + (size_t)t * p.num_heads * p.row;
    for (int e = threadIdx.x; e < p.num_heads * half; e += blockDim.x) {
        const int h = e / half, i = e % half;
        const float a = to_f32(q[h * qh + p.head_dim + 2 * i]), bb = to_f32(q[h * qh + p.head_dim + 2 * i + 1]);
        const float cs = cs_sn[i], sn = cs_sn[half + i];
        out[h * p.row + p.kv_rank + 2 * i] = from_f32<T>(a * cs - bb * sn);
        out[h * p.row + p.kv_rank + 2 * i + 1] = from_f32<T>(bb * cs + a * sn);
    }
    if (p.q_sorted_out) {
        T* sorted = (T*)p.q_sorted_out;
        for (int e = threadIdx.x; e < p.num_heads * p.head_dim; e += blockDim.x) {
            const int h = e / p.head_dim, i = e % p.head_dim;
            sorted[((size_t)h * p.n_tokens + t) * p.head_dim + i] = q[h * qh + i];
        }
    }
    const int pad = p.row - p.kv_rank - p.rot_dim;
    for (int e = threadIdx.x; e < p.num_heads * pad; e += blockDim.x)
        out[(e / pad) * p.row + p.kv_rank + p.rot_dim + e % pad] = from_f32<T>(0.f);
    for (int h = threadIdx.x; h < p.num_heads; h += blockDim.x) p.rows_out[(size_t)h * p.n_tokens + t] = t * p.num_heads + h;
    if (t == 0)
        for (int h = threadIdx.x; h <= p.num_heads; h += blockDim.x) p.offsets_out[h] = h * p.n_tokens;
}

}  // namespace

SPITE_API int spite_latent_prepare(int dtype, const LatentPrepareParams* p, const StepTokens* b, const PagedCache* c,
                                   void* stream) {
    if (!p || !b || !c || !p->down || !p->cq_out || !p->q_gain || !p->kv_gain || !p->inv_freq) return SPITE_BAD_ARG;
    if (!b->positions || !b->seg_of_token || !b->block_table || !c->kv) return SPITE_BAD_ARG;
    if (b->n_tokens < 0 || b->table_width < 1 || c->n_pages < 1 || c->page_size < 1 || c->num_kv_heads != 1) return SPITE_BAD_ARG;
    if (p->q_rank < 1 || p->kv_rank < 1 || p->rot_dim < 2 || p->rot_dim % 2 || p->num_gates < 0) return SPITE_BAD_ARG;
    if (p->gates_out ? p->num_gates < 1 : false) return SPITE_BAD_ARG;
    if (p->down_stride < (long long)p->q_rank + p->kv_rank + p->rot_dim + (p->gates_out ? p->num_gates : 0)) return SPITE_BAD_ARG;
    if (c->head_dim < p->kv_rank + p->rot_dim) return SPITE_BAD_ARG;
    if (b->n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SPITE_DT_F32) SPITE_LAUNCH(latent_prepare_kernel<float>, b->n_tokens, 256, 0, st, *p, *b, *c);
    else if (dtype == SPITE_DT_BF16) SPITE_LAUNCH(latent_prepare_kernel<__nv_bfloat16>, b->n_tokens, 256, 0, st, *p, *b, *c);
    else return SPITE_BAD_ARG;
    return spite_launch_status();
}

SPITE_API int spite_latent_queries(int dtype, const LatentQueryParams* p, void* stream) {
    if (!p || !p->q || !p->q_out || !p->inv_freq || !p->positions || !p->rows_out || !p->offsets_out) return SPITE_BAD_ARG;
    if (p->num_heads < 1 || p->head_dim < 1 || p->kv_rank < 1 || p->rot_dim < 2 || p->rot_dim % 2 || p->n_tokens < 0) return SPITE_BAD_ARG;
    if (p->row < p->kv_rank + p->rot_dim) return SPITE_BAD_ARG;
    if (p->rot_dim > 8192) return SPITE_UNSUPPORTED;
    if (p->n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)p->rot_dim * sizeof(float);
    if (dtype == SPITE_DT_F32) SPITE_LAUNCH(latent_queries_kernel<float>, p->n_tokens, 128, smem, st, *p);
    else if (dtype == SPITE_DT_BF16) SPITE_LAUNCH(latent_queries_kernel<__nv_bfloat16>, p->n_tokens, 128, smem, st, *p);
    else return SPITE_BAD_ARG;
    return spite_launch_status();
}
