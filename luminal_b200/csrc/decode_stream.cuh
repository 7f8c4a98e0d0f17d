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
#define DS_CONSUMER_WARPS 8
#define DS_CONSUMER_THREADS (32 * DS_CONSUMER_WARPS)
#define DS_THREADS (32 + DS_CONSUMER_THREADS)      // warp 0 streams weights, warps 1..8 compute
#define DS_MAX_STAGES 24
#define DS_ATTN_TILE 256

enum { DS_QKV = 0, DS_ATTN = 1, DS_O = 2, DS_GATEUP = 3, DS_DOWN = 4, DS_HEAD = 5 };

struct DsPhase {
    const unsigned char* w;      // packed units of this phase's matrix, group-major, k-slice-minor (null for DS_ATTN)
    const float* norm_w;         // RMSNorm weight folded into the staging of x, or null
    int kind, layer;
    int K, S;                    // reduction length and its number of 512-wide slices
    int groups;                  // 16-row groups of the (virtual) matrix
    int pad;
};

struct DsParams {
    const DsPhase* phases;
    int nphases, nbarriers;      // grid barriers per launch (one after every phase but the last)
    KvView kv;
    int max_seqs, max_rows;
    const int32_t* rows;         // ids | seq | pos | ctx, each [max_rows]; row 0 is the token of this step
    const float* embed;          // f32 [vocab][H]
    float *xres, *qkv, *attn, *mid, *logits;
    float* part;                 // [grid][32]: partial sums of a 16-row group that is split between CTAs
    float* attn_part;            // [nq][nsplit][130]: split attention partials (o[128], max, sum)
    unsigned long long* ctr;     // [0] grid-barrier arrivals, [1] launches completed, [2] abort; [8 + cta] split-group flags
    int H, nq, nkv, ffn, vocab;
    int nsplit, nstages, kmax;
    float eps, scale;
    RopeFreqs freqs;
    int* err;
};

size_t blum_ds_smem_bytes(int nstages, int kmax);
int blum_ds_pack(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, unsigned char* out);
size_t blum_ds_packed_bytes(int64_t rows_total, int64_t K);
int blum_ds_launch(blum_ctx* ctx, const DsParams& p);
