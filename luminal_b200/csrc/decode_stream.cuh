// Shared between decode_stream.cu (kernel + packing) and llama.cu (the model object that owns a plan).
#pragma once
#include "kv.cuh"

// One unit of the weight stream: 16 weight rows x 512 k = 16 Q8_0 blocks per row.
//   bytes [0, 8192):   16 fragments of 512 bytes, fragment j = the 16 rows' block j laid out as the A operand of
//                      mma.m16n8k32 wants it: lane l = 4*g + c holds 16 bytes
//                        W[g][8c..8c+3], W[g+8][8c..8c+3], W[g][8c+4..8c+7], W[g+8][8c+4..8c+7]   (k within block j)
//   bytes [8192, 8704): f16 block scales [16 rows][16 blocks]
#define DS_UNIT_ROWS 16
#define DS_UNIT_K 512
#define DS_UNIT_BLOCKS 16
#define DS_UNIT_BYTES 8704
#define DS_WARPS 16
#define DS_THREADS (32 * DS_WARPS)
#define DS_STAGES DS_WARPS                          // one ring stage per warp
#define DS_MAX_PHASES 448                           // 5 per layer + the head: up to 89 layers
#define DS_ATTN_TILE 256

#define DS_PARTIAL_SLOTS 128                        // per-unit row sums in flight (power of two; > ring stages + 2 * warps + slices per group)
#define DS_MAX_SLICES 64                            // K / 512 of the widest matrix
#define DS_PREFETCH_UNITS 2                         // units per warp pulled into L2 at the start of a phase

enum { DS_QKV = 0, DS_ATTN = 1, DS_O = 2, DS_GATEUP = 3, DS_DOWN = 4, DS_HEAD = 5 };

struct DsPhase {
    const unsigned char* w;      // packed units of this phase's matrix, group-major, k-slice-minor (null for DS_ATTN)
    const float* norm_w;         // RMSNorm weight folded into the staging of x, or null
    int kind, layer;
    int K, S;                    // reduction length and its number of 512-wide slices
    int groups;                  // 16-row groups of the (virtual) matrix
    int whole;                   // 1: CTAs get whole groups (no group is cut between CTAs)
};

struct DsParams {
    const DsPhase* phases;
    int nphases;
    KvView kv;
    int max_seqs, max_rows;
    int32_t* rows;               // ids | seq | pos | ctx, each [max_rows]; row 0 is the token of this step
    const float* embed;          // f32 [vocab][H]
    // activations that cross CTAs: 64-bit words {f32 value, tag of the launch and phase that wrote it}
    unsigned long long *xres, *qkv, *attn, *mid;
    unsigned long long* amax;        // [grid][2]: every CTA's (largest logit as an ordered key, its row) of the head phase
    unsigned long long* part;        // [grid][16]: partial sums of a 16-row group that is split between CTAs
    unsigned long long* attn_part;   // [nq][nsplit][130]: split attention partials (o[128], max, sum)
    float* logits;
    unsigned long long* ctr;     // [1] launches completed, [2] abort, [3..6] where the first wait gave up
    int H, nq, nkv, ffn, vocab;
    int nsplit, kmax;
    float eps, scale;
    RopeFreqs freqs;
    int* err;
    long long* prof;             // development aid: per-CTA cycle counters [grid][32] + one layer's timeline [grid][64], or null
    int prof_layer;
    // next-token choice inside the kernel (the reference's greedy rule): 0 off, 1 next[0] = argmax(logits), 2 also feeds the
    // token back into rows (token, position + 1, context + 1) and records it in hist[hist_step]
    int pick;
    int32_t* next;
    int32_t* hist;
    int hist_step;
};

size_t blum_ds_smem_bytes(int kmax);
int blum_ds_pack(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, unsigned char* out);
size_t blum_ds_packed_bytes(int64_t rows_total, int64_t K);
int blum_ds_launch(blum_ctx* ctx, const DsParams& p);

// prompt-chunk matmul over the same packed units (prefill_rows.cu)
size_t blum_rows_scratch_bytes(int M, int64_t K_max, int64_t nk_max);
int blum_rows_matmul(blum_ctx* ctx, const unsigned char* packed, int64_t rows_total, int64_t K, const void* x, int xdt, int64_t ldx, int M,
                     int swiglu, void* y, int ydt, int64_t ldy, void* scratch, size_t scratch_bytes);
