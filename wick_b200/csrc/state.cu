// The per-sequence state record on the device, and the kernels that let a batch
// decode step after step without the host in between.
//
// A record is 8 int32 words, one record per cache slot (slot 0 is the padding
// slot: its record stays zero apart from "finished", so a padded row runs token
// 0 at position 0 of the reserved page for ever):
//   [0] length       positions the cache holds = the position of the next token
//   [1] next_token   the token the next step feeds (the one sampled last)
//   [2] finished     0 running, 1 a stop token was sampled, 2 the limit is reached
//   [3] n_generated  tokens sampled so far (a stop token counts)
//   [4] limit        tokens this sequence may generate
//   [5] row          the sequence's row in its batch's sampler state (generator, seen tokens)
//
// step_prepare turns records into the fields of a decode step's batch
// description (token, position, cached length before and after); step_advance
// takes the sampled ids, decides who is finished (wick src/engine.rs:178-206: a
// stop token ends the sequence and is never fed; the length limit ends it after
// the token is kept) and moves the others on.  A finished sequence is frozen:
// while it still rides along in a batch it runs its last step again and again,
// which writes the same key and value to the same place and changes nothing.
#include "common.cuh"
#include "sm100.cuh"

namespace wick {

constexpr int REC = 8;
enum { F_LENGTH = 0, F_NEXT = 1, F_FINISHED = 2, F_GENERATED = 3, F_LIMIT = 4, F_ROW = 5 };

__global__ void seq_state_set_kernel(int* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ values, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * REC) return;
    state[(int64_t)slots[i / REC] * REC + i % REC] = values[i];
}

// (This kernel never lets its successor start early: kernels further down the step read the
// fields it writes, the lengths among them, before they wait for their own predecessor, as
// they may with a description that the host has copied in.  With no early start here, every
// kernel of the step begins after these fields are complete.)
__global__ void step_prepare_kernel(const int* state, const int* __restrict__ slots, int* __restrict__ tokens,
                                    int* __restrict__ positions, int* __restrict__ start, int* __restrict__ kv_len, int n) {
    pdl_wait();
    state = fresh(state);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int* r = state + (int64_t)slots[i] * REC;
    const int len = r[F_LENGTH];
    tokens[i] = r[F_NEXT];
    positions[i] = len;
    start[i] = len;
    kv_len[i] = len + 1;
}

// ids: the tokens sampled for the step's rows; kv_len: the cached length of each row after
// the step; seen: [rows of the batch, vocab] bytes (or null), 1 where a token has occurred.
// ids[n] receives the device status word, so that the host reads both with one copy.
__global__ void step_advance_kernel(int* state, const int* __restrict__ slots, int* ids, const int* kv_len,
                                    const int* __restrict__ stops, int n_stops, uint8_t* __restrict__ seen, int vocab,
                                    const int* status, int n) {
    pdl_trigger();
    pdl_wait();
    ids = fresh(ids);
    kv_len = fresh(kv_len);
    state = fresh(state);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) ids[n] = status ? *status : 0;
    if (i >= n) return;
    const int slot = slots[i];
    if (slot == 0) return;
    int* r = state + (int64_t)slot * REC;
    if (r[F_FINISHED]) return;
    const int tok = ids[i];
    const int made = r[F_GENERATED] + 1;
    r[F_GENERATED] = made;
    r[F_LENGTH] = kv_len[i];
    r[F_NEXT] = tok;
    bool stop = false;
    for (int k = 0; k < n_stops; ++k) stop |= stops[k] == tok;
    if (stop)
        r[F_FINISHED] = 1;
    else {
        if (made >= r[F_LIMIT]) r[F_FINISHED] = 2;
        if (seen && tok >= 0 && tok < vocab) seen[(int64_t)r[F_ROW] * vocab + tok] = 1;
    }
}

// xoshiro256** (wick src/sampler.rs:29-61): one generator per row of the batch's sampler
// state, one 24-bit uniform number per step for every row that is still running.
__device__ __forceinline__ uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

__global__ void rng_uniforms_kernel(uint64_t* __restrict__ rng, const int* state, const int* __restrict__ slots,
                                    float* __restrict__ out, int n) {
    pdl_trigger();
    pdl_wait();
    state = fresh(state);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int* r = state + (int64_t)slots[i] * REC;
    if (slots[i] == 0 || r[F_FINISHED]) {
        out[i] = 0.f;
        return;
    }
    uint64_t* s = rng + (int64_t)r[F_ROW] * 4;
    const uint64_t result = rotl64(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    out[i] = (float)(result >> 40) / (float)(1 << 24);
}

// The tokens of a prompt step, marked as seen in their sequences' rows.
__global__ void seen_prompt_kernel(uint8_t* __restrict__ seen, int vocab, const int* state, const int* __restrict__ slots,
                                   const int* __restrict__ tokens, const int* __restrict__ seq_of_token, int n_tokens) {
    pdl_trigger();
    pdl_wait();
    state = fresh(state);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens) return;
    const int slot = slots[seq_of_token[i]];
    const int tok = tokens[i];
    if (slot == 0 || tok < 0 || tok >= vocab) return;
    seen[(int64_t)state[(int64_t)slot * REC + F_ROW] * vocab + tok] = 1;
}

// wick src/sampler.rs:76-85 over the seen-token table: a seen token's logit is divided by
// the penalty if positive, multiplied otherwise.
__global__ void penalty_seen_kernel(float* logits, const uint8_t* __restrict__ seen, int vocab, const int* state,
                                    const int* __restrict__ slots, float penalty, int n) {
    pdl_trigger();
    pdl_wait();
    logits = fresh(logits);
    state = fresh(state);
    const int row = blockIdx.y;
    const int slot = slots[row];
    if (slot == 0) return;
    const uint8_t* mine = seen + (int64_t)state[(int64_t)slot * REC + F_ROW] * vocab;
    float* x = logits + (int64_t)row * vocab;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < vocab; v += gridDim.x * blockDim.x) {
        if (mine[v]) {
            const float l = x[v];
            x[v] = l > 0.f ? l / penalty : l * penalty;
        }
    }
}

// A kernel whose only wait can never be satisfied: one block, one mbarrier that nothing
// arrives on, no copy in flight.  It goes through the same bounded wait as every ring kernel
// (sm100.cuh: mbar_wait), gives up after limit_ns, leaves its code in the status word and
// returns.  It exists so that a test can see the give-up path end to end.
__global__ void wait_gives_up_kernel(int* status, int code, uint64_t limit_ns, int* gave_up) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait(&bar, 0, &abort_flag, status, code, limit_ns);
        *gave_up = ok ? 0 : 1;
    }
}

}  // namespace wick

using namespace wick;

WICK_API int wick_wait_gives_up(int* status, int code, long long limit_ns, int* gave_up, void* s) {
    WICK_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, "wait_gives_up: the limit must lie within 100 ms");
    wait_gives_up_kernel<<<1, 32, 0, (cudaStream_t)s>>>(status, code, (uint64_t)limit_ns, gave_up);
    return check_launch("wait_gives_up");
}

WICK_API int wick_seq_state_words() { return REC; }

WICK_API int wick_seq_state_set(int* state, const int* slots, const int* values, int n, void* s) {
    if (n <= 0) return 0;
    WICK_CUDA(launch(seq_state_set_kernel, dim3(ceil_div((int64_t)n * REC, 256)), dim3(256), 0, (cudaStream_t)s, state, slots, values, n));
    return check_launch("seq_state_set");
}

WICK_API int wick_step_prepare(const int* state, const int* slots, int* tokens, int* positions, int* start, int* kv_len, int n,
                               void* s) {
    if (n <= 0) return 0;
    WICK_CUDA(launch(step_prepare_kernel, dim3(ceil_div(n, 128)), dim3(128), 0, (cudaStream_t)s, state, slots, tokens, positions,
                     start, kv_len, n));
    return check_launch("step_prepare");
}

WICK_API int wick_step_advance(int* state, const int* slots, int* ids, const int* kv_len, const int* stops, int n_stops,
                               void* seen, int vocab, const int* status, int n, void* s) {
    WICK_REQUIRE(n >= 1, "step_advance: no rows");
    WICK_CUDA(launch(step_advance_kernel, dim3(ceil_div(n, 128)), dim3(128), 0, (cudaStream_t)s, state, slots, ids, kv_len, stops,
                     n_stops, (uint8_t*)seen, vocab, status, n));
    return check_launch("step_advance");
}

WICK_API int wick_rng_uniforms(void* rng, const int* state, const int* slots, float* out, int n, void* s) {
    if (n <= 0) return 0;
    WICK_CUDA(launch(rng_uniforms_kernel, dim3(ceil_div(n, 128)), dim3(128), 0, (cudaStream_t)s, (uint64_t*)rng, state, slots, out, n));
    return check_launch("rng_uniforms");
}

WICK_API int wick_seen_prompt(void* seen, int vocab, const int* state, const int* slots, const int* tokens,
                              const int* seq_of_token, int n_tokens, void* s) {
    if (n_tokens <= 0) return 0;
    WICK_CUDA(launch(seen_prompt_kernel, dim3(ceil_div(n_tokens, 256)), dim3(256), 0, (cudaStream_t)s, (uint8_t*)seen, vocab, state,
                     slots, tokens, seq_of_token, n_tokens));
    return check_launch("seen_prompt");
}

WICK_API int wick_penalty_seen(float* logits, const void* seen, int vocab, const int* state, const int* slots, float penalty,
                               int n, void* s) {
    if (n <= 0) return 0;
    WICK_CUDA(launch(penalty_seen_kernel, dim3(min(64, ceil_div(vocab, 256)), n), dim3(256), 0, (cudaStream_t)s, logits,
                     (const uint8_t*)seen, vocab, state, slots, penalty, n));
    return check_launch("penalty_seen");
}
