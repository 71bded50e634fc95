// Between two decode steps that run back to back on the device: the sampled
// token becomes the next input, every request moves one position on, and the
// slot of the new position is looked up in the block table.  It lets several
// decode steps run without the host in between (the pages for them are
// reserved beforehand).  The reference's loop goes through the host every
// step (crates/vllm-engine/src/engine.rs:82-163).
#include "common.cuh"

__global__ void decode_advance_kernel(int* __restrict__ token_ids, const int* __restrict__ sampled,
                                      int* __restrict__ positions, int* __restrict__ context_lens,
                                      int* __restrict__ start_pos, int* __restrict__ slots,
                                      const int* __restrict__ block_table, int max_blocks, int page_size, int B,
                                      int* __restrict__ out_tokens, int* __restrict__ step_counter, int max_steps) {
    pdl_wait();
    pdl_trigger();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int step = *step_counter;
    const int tok = sampled[b];
    if (step < max_steps) out_tokens[(size_t)step * B + b] = tok;
    token_ids[b] = tok;
    const int pos = positions[b] + 1;
    positions[b] = pos;
    context_lens[b] = pos + 1;
    start_pos[b] = pos;
    const int blk = pos / page_size;
    // beyond the reserved pages nothing is written (slot -1); the host never runs that far
    slots[b] = blk < max_blocks ? block_table[(size_t)b * max_blocks + blk] * page_size + pos % page_size : -1;
}

__global__ void bump_counter_kernel(int* c) {
    pdl_wait();
    pdl_trigger();
    *c += 1;
}

extern "C" int rg_decode_advance(int* token_ids, const int* sampled, int* positions, int* context_lens,
                                 int* start_pos, int* slots, const int* block_table, int max_blocks,
                                 int page_size, int B, int* out_tokens, int* step_counter, int max_steps,
                                 void* stream) {
    if (B <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int e = rg_launch(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s, 1, token_ids, sampled, positions,
                      context_lens, start_pos, slots, block_table, max_blocks, page_size, B, out_tokens, step_counter,
                      max_steps);
    if (e) return e;
    return rg_launch(bump_counter_kernel, dim3(1), dim3(1), 0, s, 1, step_counter);
}
