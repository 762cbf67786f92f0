// A selective state-space recurrence with a short causal convolution in front of it (the "state-space
// duality" layer): per head h (with its group g of B and C)
//     dt_t = softplus(raw_t + dt_bias_h);   S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T;   y_t = S_t^T C_t + D_h x_t
// with S [N, P] float32 per (request, head), kept in the request's state slot between steps, and in front of
// it, per channel c of (x | B | C):  u_t = silu(bias_c + sum_k w[c, k] in_(t - (taps - 1 - k))), zeros before the
// sequence's start; the last taps - 1 inputs of a request are part of its state too.
//
// Everything here is float32.  A request's rows are contiguous in a step; where a sequence starts at position 0
// its state counts as zero, whatever the slot held (slots are used again).  State slot -1: a padding sequence,
// nothing is read or written.  The step's facts come from device arrays only, so a step can be recorded.
#include "common.cuh"

#define SSM_MAX_TAPS 16
#define SSM_PER_LANE 16         // state rows (of N) a thread keeps in registers

// in [tokens, in_stride] float32, the channels at column `offset`; conv_state [slots, (taps - 1), channels] with
// `state_stride` floats from slot to slot; out [tokens, channels].
// A thread keeps one channel and walks down SSM_CONV_ROWS rows with the last taps - 1 inputs in registers: where a row
// follows the row before it in the same sequence, one input is loaded for it; at the block's first row and at a
// sequence's first row of the step the inputs before it come from the rows above or from the slot's state.
#define SSM_CONV_ROWS 16

template <int MAX_TAPS>
__global__ void causal_conv_silu_kernel(const float* __restrict__ in, int in_stride, int offset, const float* __restrict__ weight,
                                        const float* __restrict__ bias, const float* __restrict__ conv_state, long long state_stride,
                                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                        const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                        float* __restrict__ out, int tokens, int channels, int taps, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first = blockIdx.x * rows, last = min(tokens, first + rows);
    float w[MAX_TAPS], history[MAX_TAPS];          // history[j]: the input taps - 1 - j rows back, j < taps - 1
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) w[k] = k < taps ? weight[(size_t)c * taps + k] : 0.0f;
    const float b = bias ? bias[c] : 0.0f;
    int previous_seq = -1;
    for (int t = first; t < last; ++t) {
        const int seq = seq_of_token[t];
        const int start_row = q_start[seq], end_row = q_start[seq + 1];
        const int slot = state_slots[seq];
        if (t < start_row || t >= end_row || slot < 0) {          // a padding row
            out[(size_t)t * channels + c] = 0.0f;
            previous_seq = -1;
            continue;
        }
        const int pos = positions[t];
        if (seq != previous_seq || t == start_row) {              // the inputs before this row, afresh
            const float* state = conv_state + (long long)slot * state_stride;
#pragma unroll
            for (int j = 0; j < MAX_TAPS - 1; ++j) {
                const int back = taps - 1 - j, row = t - back;
                float x = 0.0f;
                if (j < taps - 1 && pos - back >= 0) x = row >= start_row ? in[(size_t)row * in_stride + offset + c]
                                                          : state[(size_t)(taps - 1 - (start_row - row)) * channels + c];
                history[j] = x;
            }
            previous_seq = seq;
        }
        const float now = in[(size_t)t * in_stride + offset + c];
        float acc = b;
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            if (j < taps - 1) acc += w[j] * history[j];
            else if (j == taps - 1) acc += w[j] * now;
        }
#pragma unroll
        for (int j = 0; j < MAX_TAPS - 1; ++j) {
            if (j < taps - 2) history[j] = history[j + 1];
            else if (j == taps - 2) history[j] = now;
        }
        out[(size_t)t * channels + c] = acc / (1.0f + expf(-acc));
    }
}

// After the convolution has read the old state: the last taps - 1 inputs of every sequence become its state.
__global__ void conv_state_update_kernel(const float* __restrict__ in, int in_stride, int offset, float* __restrict__ conv_state,
                                         long long state_stride, const int* __restrict__ positions, const int* __restrict__ q_start,
                                         const int* __restrict__ state_slots, int channels, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x;
    const int start_row = q_start[seq], n = q_start[seq + 1] - start_row;
    const int slot = state_slots[seq];
    if (slot < 0 || n <= 0) return;
    const int start_pos = positions[start_row];
    float* state = conv_state + (long long)slot * state_stride;
    const int keep = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float next[SSM_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < SSM_MAX_TAPS; ++j) {
            if (j >= keep) break;
            const int rel = n - keep + j;                 // row of the portion that lands in place j
            if (rel >= 0) next[j] = in[(size_t)(start_row + rel) * in_stride + offset + c];
            else next[j] = start_pos + rel >= 0 ? state[(size_t)(j + n) * channels + c] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < SSM_MAX_TAPS; ++j) {
            if (j >= keep) break;
            state[(size_t)j * channels + c] = next[j];
        }
    }
}

MRS_EXPORT int mrs_causal_conv_silu(const float* in, int in_stride, int offset, const float* weight, const float* bias,
                                    float* conv_state, long long state_stride, const int* positions, const int* seq_of_token,
                                    const int* q_start, const int* state_slots, float* out, int tokens, int sequences, int channels,
                                    int taps, int update_state, void* stream) {
    if (tokens <= 0) return 0;
    if (channels <= 0 || taps <= 0 || taps > SSM_MAX_TAPS) return MRS_BAD_ARGUMENT;
    const int threads = 128;
    const int across = (channels + threads - 1) / threads;
    int per_row = across > 64 ? 64 : across;               // the state update strides over the channels
    if (across > 65535) return MRS_BAD_ARGUMENT;
    const int rows = tokens >= 32 * SSM_CONV_ROWS ? SSM_CONV_ROWS : 1;      // few rows (decoded tokens): a thread a row
    const dim3 grid((tokens + rows - 1) / rows, across);
    if (taps <= 4)
        MRS_LAUNCH(causal_conv_silu_kernel<4>, grid, threads, 0, stream, in, in_stride, offset, weight, bias, (const float*)conv_state,
                   state_stride, positions, seq_of_token, q_start, state_slots, out, tokens, channels, taps, rows);
    else if (taps <= 8)
        MRS_LAUNCH(causal_conv_silu_kernel<8>, grid, threads, 0, stream, in, in_stride, offset, weight, bias, (const float*)conv_state,
                   state_stride, positions, seq_of_token, q_start, state_slots, out, tokens, channels, taps, rows);
    else
        MRS_LAUNCH(causal_conv_silu_kernel<SSM_MAX_TAPS>, grid, threads, 0, stream, in, in_stride, offset, weight, bias,
                   (const float*)conv_state, state_stride, positions, seq_of_token, q_start, state_slots, out, tokens, channels, taps, rows);
    if (update_state && taps > 1)
        MRS_LAUNCH(conv_state_update_kernel, dim3(sequences, per_row), threads, 0, stream, in, in_stride, offset, conv_state,
                   state_stride, positions, q_start, state_slots, channels, taps);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// The recurrence, token by token.  One block per (sequence, head, slice of the head's columns); thread (p, s): column p
// of S (SSM_COLUMNS neighbouring ones) and the rows n = s * per + i of it in registers (lanes of one p are neighbours, so that y's sum over n is a few shuffles).
// xbc [tokens, heads * P + 2 * groups * N] float32 (x | B | C after convolution and silu), raw dt a column range of
// the projection's rows, y [tokens, heads * P] float32.  ssm_state [slots, heads, N, P].
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

// WHOLE: a sequence's rows in one go, from the slot's state to the slot's state.  For long portions the rows are cut
// into chunks of `chunk_len` that run side by side in three passes: LOCAL runs every chunk from a zero state and leaves
// its end state and the product of its decays in scratch; `ssm_chunk_states_kernel` walks a sequence's chunks once,
// turning the local end states into the true state at every chunk's start (and the slot's new state); FINAL runs every
// chunk again from that state and writes y.
enum { SSM_WHOLE = 0, SSM_LOCAL = 1, SSM_FINAL = 2 };

// Rows are taken SSM_BATCH at a time (fewer where the state is large): their B, C and x come into shared memory by
// asynchronous copies, the step sizes and decays are computed once a row (not once a warp), and every thread walks them
// while the next batch's copies are in flight.  In shared memory a row's B (and C) lie as [i / 4][s][i % 4] for the element n = s * per + i,
// padded with zeros to 16 elements a lane: a thread reads its 16 values as four vectors, and the lanes of a warp read
// neighbouring vectors.
#define SSM_BATCH 16
#define SSM_COLUMNS 1           // columns of S a thread owns (two were measured and are slower: 518 against 446 us for 2,048 rows in chunks)

__device__ __forceinline__ void cp_async_f4(float* to, const float* from) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(to)), "l"(from));
}
__device__ __forceinline__ void cp_async_f1(float* to, const float* from) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(to)), "l"(from));
}

template <int MODE, int LANES>
__global__ void ssm_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ dt_in, int dt_stride,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                                float* __restrict__ ssm_state, long long state_stride, const int* __restrict__ positions,
                                const int* __restrict__ q_start, const int* __restrict__ state_slots, float* __restrict__ y,
                                int heads, int groups, int N, int P, int per, int write_state,
                                float* __restrict__ chunk_state, float* __restrict__ chunk_decay, int chunk_len, int max_chunks,
                                int slices, int columns, int batch) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int lanes_per_column = LANES;                          // lanes that share a column of S (a power of two)
    extern __shared__ __align__(16) float ssm_smem[];
    const int seq = blockIdx.x, head = blockIdx.y / slices, slice = blockIdx.y % slices, chunk = blockIdx.z;
    const int seq_start = q_start[seq], seq_end = q_start[seq + 1];
    const int slot = state_slots[seq];
    if (slot < 0 || seq_end <= seq_start) return;
    const int start_row = MODE == SSM_WHOLE ? seq_start : seq_start + chunk * chunk_len;
    const int end_row = MODE == SSM_WHOLE ? seq_end : min(seq_end, start_row + chunk_len);
    if (start_row >= end_row) return;
    // a thread owns SSM_COLUMNS neighbouring columns: what it reads of B and C serves them all
    const int s = threadIdx.x % lanes_per_column, column = (threadIdx.x / lanes_per_column) * SSM_COLUMNS, p = slice * columns + column;
    bool live[SSM_COLUMNS];
#pragma unroll
    for (int j = 0; j < SSM_COLUMNS; ++j) live[j] = p + j < P && column + j < columns;
    const int group = head / (heads / groups);
    const int inner = heads * P, row_width = inner + 2 * groups * N;
    const int n0 = s * per;
    const int padded = SSM_PER_LANE * lanes_per_column;              // floats of a row's B (or C) in shared memory
    float* b_rows = ssm_smem;                                        // [2][batch][padded]
    float* c_rows = b_rows + (size_t)2 * batch * padded;             // [2][batch][padded]
    float* x_rows = c_rows + (size_t)2 * batch * padded;             // [2][batch][columns]
    float* dt_rows = x_rows + (size_t)2 * batch * columns;           // [2][batch] step sizes
    float* decay_rows = dt_rows + 2 * batch;                         // [2][batch] decays
    const int rows_here = end_row - start_row;                       // the padding of the rows in use stays zero
    const int used = (rows_here > batch ? 2 * batch : rows_here) * padded;
    for (int i = threadIdx.x; i < used; i += blockDim.x) b_rows[i] = 0.0f, c_rows[i] = 0.0f;

    float* state = MODE == SSM_WHOLE ? ssm_state + (long long)slot * state_stride + (size_t)head * N * P
                                     : chunk_state + (((size_t)seq * heads + head) * max_chunks + chunk) * N * P;
    float S[SSM_COLUMNS][SSM_PER_LANE];
    const bool zero = MODE == SSM_LOCAL || (MODE == SSM_WHOLE && positions[seq_start] == 0);
#pragma unroll
    for (int j = 0; j < SSM_COLUMNS; ++j)
#pragma unroll
        for (int i = 0; i < SSM_PER_LANE; ++i)
            S[j][i] = (!zero && live[j] && i < per && n0 + i < N) ? state[(size_t)(n0 + i) * P + p + j] : 0.0f;
    const float bias = dt_bias[head], rate = -expf(a_log[head]), skip = d_skip[head];
    float decays = 1.0f;

    // Two buffers: while the threads walk one batch of rows, the copies of the next are in flight (cp.async, 16 bytes
    // where the sizes allow it), and the step sizes of the next batch wait in a register.
    const bool vectors = per % 4 == 0 && N % 4 == 0 && row_width % 4 == 0 && (inner + group * N) % 4 == 0 && (groups * N) % 4 == 0 &&
                         (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
    auto fetch = [&](int buffer, int first, int count) {
        float* b_to = b_rows + (size_t)buffer * batch * padded;
        float* c_to = c_rows + (size_t)buffer * batch * padded;
        float* x_to = x_rows + (size_t)buffer * batch * columns;
        if (vectors && blockDim.x % (N / 4) == 0) {
            // a thread's place in a row is the same in every pass of the loop: the divisions are done once
            const int quads = N / 4, n = ((int)threadIdx.x % quads) * 4, step = blockDim.x / quads;
            const int where = ((((n % per) >> 2) * lanes_per_column + n / per) << 2);
            const float* r = xbc + (size_t)first * row_width + inner + group * N + n;
            for (int t = threadIdx.x / quads; t < count; t += step) {
                cp_async_f4(b_to + t * padded + where, r + (size_t)t * row_width);
                if (MODE != SSM_LOCAL) cp_async_f4(c_to + t * padded + where, r + (size_t)t * row_width + groups * N);
            }
        } else if (vectors) {
            const int quads = N / 4;
            for (int i = threadIdx.x; i < count * quads; i += blockDim.x) {
                const int t = i / quads, n = (i % quads) * 4;
                const float* r = xbc + (size_t)(first + t) * row_width + inner + group * N + n;
                const int where = t * padded + ((((n % per) >> 2) * lanes_per_column + n / per) << 2);
                cp_async_f4(b_to + where, r);
                if (MODE != SSM_LOCAL) cp_async_f4(c_to + where, r + groups * N);
            }
        } else {
            for (int i = threadIdx.x; i < count * N; i += blockDim.x) {
                const int t = i / N, n = i % N;
                const float* r = xbc + (size_t)(first + t) * row_width + inner + group * N + n;
                const int at = n % per;
                const int where = t * padded + (((at >> 2) * lanes_per_column + n / per) << 2) + (at & 3);
                cp_async_f1(b_to + where, r);
                if (MODE != SSM_LOCAL) cp_async_f1(c_to + where, r + groups * N);
            }
        }
        if (blockDim.x % columns == 0) {
            const int c = (int)threadIdx.x % columns, step = blockDim.x / columns;
            for (int t = threadIdx.x / columns; t < count; t += step) {
                if (slice * columns + c < P) cp_async_f1(x_to + t * columns + c, xbc + (size_t)(first + t) * row_width + head * P + slice * columns + c);
                else x_to[t * columns + c] = 0.0f;
            }
        } else {
            for (int i = threadIdx.x; i < count * columns; i += blockDim.x) {
                const int t = i / columns, c = i % columns;
                if (slice * columns + c < P) cp_async_f1(x_to + i, xbc + (size_t)(first + t) * row_width + head * P + slice * columns + c);
                else x_to[i] = 0.0f;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    auto step_sizes = [&](int buffer, int count, float raw) {
        if ((int)threadIdx.x < count) {
            const float dt = softplus_f(raw + bias);
            dt_rows[buffer * batch + threadIdx.x] = dt;
            decay_rows[buffer * batch + threadIdx.x] = expf(rate * dt);
        }
    };
    {
        const int count = min(batch, end_row - start_row);
        __syncthreads();                                             // the zeros are written
        fetch(0, start_row, count);
        step_sizes(0, count, (int)threadIdx.x < count ? dt_in[(size_t)(start_row + threadIdx.x) * dt_stride + head] : 0.0f);
    }
    int buffer = 0;
    for (int first = start_row; first < end_row; first += batch, buffer ^= 1) {
        const int count = min(batch, end_row - first);
        const int next_count = min(batch, end_row - (first + batch));
        float next_raw = 0.0f;
        if (next_count > 0) {
            fetch(buffer ^ 1, first + batch, next_count);
            if ((int)threadIdx.x < next_count) next_raw = dt_in[(size_t)(first + batch + threadIdx.x) * dt_stride + head];
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const float* b_from = b_rows + (size_t)buffer * batch * padded;
        const float* c_from = c_rows + (size_t)buffer * batch * padded;
        const float* x_from = x_rows + (size_t)buffer * batch * columns;
        float* y_row = y + (size_t)first * inner + head * P + p;
        for (int t = 0; t < count; ++t) {
            const float decay = decay_rows[buffer * batch + t], dt = dt_rows[buffer * batch + t];
            float x[SSM_COLUMNS], dx[SSM_COLUMNS], sum[SSM_COLUMNS];
#pragma unroll
            for (int j = 0; j < SSM_COLUMNS; ++j) {
                x[j] = column + j < columns ? x_from[t * columns + column + j] : 0.0f;
                dx[j] = dt * x[j];
                sum[j] = 0.0f;
            }
            if (MODE == SSM_LOCAL) decays *= decay;
#pragma unroll
            for (int v = 0; v < SSM_PER_LANE / 4; ++v) {
                const float4 b = *reinterpret_cast<const float4*>(b_from + t * padded + ((v * lanes_per_column + s) << 2));
                float4 c = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (MODE != SSM_LOCAL) c = *reinterpret_cast<const float4*>(c_from + t * padded + ((v * lanes_per_column + s) << 2));
#pragma unroll
                for (int j = 0; j < SSM_COLUMNS; ++j) {
                    S[j][4 * v + 0] = decay * S[j][4 * v + 0] + dx[j] * b.x;
                    S[j][4 * v + 1] = decay * S[j][4 * v + 1] + dx[j] * b.y;
                    S[j][4 * v + 2] = decay * S[j][4 * v + 2] + dx[j] * b.z;
                    S[j][4 * v + 3] = decay * S[j][4 * v + 3] + dx[j] * b.w;
                    if (MODE != SSM_LOCAL)
                        sum[j] += S[j][4 * v + 0] * c.x + S[j][4 * v + 1] * c.y + S[j][4 * v + 2] * c.z + S[j][4 * v + 3] * c.w;
                }
            }
            if (MODE != SSM_LOCAL) {
#pragma unroll
                for (int j = 0; j < SSM_COLUMNS; ++j) {
#pragma unroll
                    for (int o = 1; o < lanes_per_column; o <<= 1) sum[j] += __shfl_xor_sync(0xffffffffu, sum[j], o);
                    if (live[j] && s == 0) y_row[j] = sum[j] + skip * x[j];
                }
                y_row += inner;
            }
        }
        step_sizes(buffer ^ 1, next_count, next_raw);
        __syncthreads();                                             // this buffer is read; the next one's step sizes are written
    }
    if (MODE == SSM_LOCAL && threadIdx.x == 0 && slice == 0) chunk_decay[((size_t)seq * heads + head) * max_chunks + chunk] = decays;
    if (MODE == SSM_LOCAL || (MODE == SSM_WHOLE && write_state)) {
#pragma unroll
        for (int j = 0; j < SSM_COLUMNS; ++j)
#pragma unroll
            for (int i = 0; i < SSM_PER_LANE; ++i)
                if (live[j] && i < per && n0 + i < N) state[(size_t)(n0 + i) * P + p + j] = S[j][i];
    }
}

// One thread an element of a (sequence, head)'s state: chunk c's entry of `chunk_state` goes from the chunk's local end
// state to the state at its start, S_in[0] = the slot's state (zero at position 0), S_in[c + 1] = decay_c S_in[c] + local_c.
__global__ void ssm_chunk_states_kernel(float* __restrict__ ssm_state, long long state_stride, const int* __restrict__ positions,
                                        const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                        float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int heads, int elements,
                                        int chunk_len, int max_chunks, int write_state) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int seq_start = q_start[seq], rows = q_start[seq + 1] - seq_start;
    const int slot = state_slots[seq];
    if (slot < 0 || rows <= 0) return;
    const int chunks = (rows + chunk_len - 1) / chunk_len;
    const bool fresh = positions[seq_start] == 0;
    float* state = ssm_state + (long long)slot * state_stride + (size_t)head * elements;
    float* local = chunk_state + ((size_t)seq * heads + head) * max_chunks * elements;
    const float* decay = chunk_decay + ((size_t)seq * heads + head) * max_chunks;
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < elements; i += gridDim.z * blockDim.x) {
        float value = fresh ? 0.0f : state[i];
        for (int c = 0; c < chunks; ++c) {
            const float end = local[(size_t)c * elements + i];
            local[(size_t)c * elements + i] = value;
            value = decay[c] * value + end;
        }
        if (write_state) state[i] = value;
    }
}

// `chunk_len` 0: every sequence in one go.  Otherwise the three passes over chunks of that many rows; `scratch` then holds
// sequences * heads * max_chunks * (N * P + 1) floats, max_chunks = ceil(tokens / chunk_len).
MRS_EXPORT int mrs_ssm_scan(const float* xbc, const float* dt_in, int dt_stride, const float* dt_bias, const float* a_log,
                            const float* d_skip, float* ssm_state, long long state_stride, const int* positions, const int* q_start,
                            const int* state_slots, float* y, int tokens, int sequences, int heads, int groups, int N, int P,
                            int write_state, int chunk_len, float* scratch, void* stream) {
    if (sequences <= 0 || tokens <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || chunk_len < 0 || (chunk_len > 0 && !scratch))
        return MRS_BAD_ARGUMENT;
    int lanes = 1;
    while (lanes < 32 && (N + lanes - 1) / lanes > SSM_PER_LANE) lanes <<= 1;
    const int per = (N + lanes - 1) / lanes;
    if (per > SSM_PER_LANE) return MRS_BAD_ARGUMENT;                 // N above 512
    // blocks of about 128 threads, each a slice of a head's columns: several blocks share an SM and hide one another's waits
    int columns = 128 / lanes;
    if (columns > P) columns = P;
    const int slices = (P + columns - 1) / columns;
    const int threads = ((columns + SSM_COLUMNS - 1) / SSM_COLUMNS * lanes + 31) / 32 * 32;
    if ((long long)heads * slices > 65535) return MRS_BAD_ARGUMENT;
    // rows a batch: what 40 KB of shared memory hold (several blocks share an SM), at least one, at most as many as threads
    const int row_floats = 2 * SSM_PER_LANE * lanes + columns + 2;
    int batch = (40 * 1024 / 4) / (2 * row_floats);       // two buffers
    if (batch > SSM_BATCH) batch = SSM_BATCH;
    if (batch > threads) batch = threads;
    if (batch < 1) batch = 1;
    const size_t smem = (size_t)2 * batch * row_floats * sizeof(float);
#define SSM_LAUNCH(MODE, LANES, GRID, STATE, DECAY, CHUNK, CHUNKS)                                                            \
    MRS_LAUNCH((ssm_scan_kernel<MODE, LANES>), GRID, threads, smem, stream, xbc, dt_in, dt_stride, dt_bias, a_log, d_skip,         \
               ssm_state, state_stride, positions, q_start, state_slots, y, heads, groups, N, P, per, write_state, STATE, DECAY,   \
               CHUNK, CHUNKS, slices, columns, batch)
#define SSM_LAUNCH_LANES(MODE, GRID, STATE, DECAY, CHUNK, CHUNKS)                                                                \
    switch (lanes) {                                                                                                               \
        case 1: SSM_LAUNCH(MODE, 1, GRID, STATE, DECAY, CHUNK, CHUNKS); break;                                                     \
        case 2: SSM_LAUNCH(MODE, 2, GRID, STATE, DECAY, CHUNK, CHUNKS); break;                                                     \
        case 4: SSM_LAUNCH(MODE, 4, GRID, STATE, DECAY, CHUNK, CHUNKS); break;                                                     \
        case 8: SSM_LAUNCH(MODE, 8, GRID, STATE, DECAY, CHUNK, CHUNKS); break;                                                     \
        case 16: SSM_LAUNCH(MODE, 16, GRID, STATE, DECAY, CHUNK, CHUNKS); break;                                                   \
        default: SSM_LAUNCH(MODE, 32, GRID, STATE, DECAY, CHUNK, CHUNKS); break;                                                   \
    }
    if (chunk_len == 0) {
        SSM_LAUNCH_LANES(SSM_WHOLE, dim3(sequences, heads * slices), (float*)nullptr, (float*)nullptr, 0, 0);
        MRS_RETURN_LAUNCH_STATUS();
    }
    const int max_chunks = (tokens + chunk_len - 1) / chunk_len;
    if (max_chunks > 65535) return MRS_BAD_ARGUMENT;
    float* chunk_state = scratch;
    float* chunk_decay = scratch + (size_t)sequences * heads * max_chunks * N * P;
    SSM_LAUNCH_LANES(SSM_LOCAL, dim3(sequences, heads * slices, max_chunks), chunk_state, chunk_decay, chunk_len, max_chunks);
    const int elements = N * P;
    int element_blocks = (elements + 255) / 256;
    if (element_blocks > 64) element_blocks = 64;
    MRS_LAUNCH(ssm_chunk_states_kernel, dim3(sequences, heads, element_blocks), 256, 0, stream, ssm_state, state_stride, positions, q_start,
               state_slots, chunk_state, (const float*)chunk_decay, heads, elements, chunk_len, max_chunks, write_state);
    SSM_LAUNCH_LANES(SSM_FINAL, dim3(sequences, heads * slices, max_chunks), chunk_state, chunk_decay, chunk_len, max_chunks);
    MRS_RETURN_LAUNCH_STATUS();
}
