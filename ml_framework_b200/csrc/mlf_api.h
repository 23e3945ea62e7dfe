// C ABI of libmlfb200.so. Every function returns 0 on success and a negative value on a
// host-side failure (message via mlf_last_error()). Kernels that give up on a bounded wait
// write a code to the per-device status word, read with mlf_read_status().
//
// All pointers are device pointers unless a comment says otherwise; `stream` is a
// cudaStream_t passed as an integer handle (0 = legacy default stream).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM epilogue flags -----------------------------------------------------------------
enum {
  MLF_EPI_BIAS = 1,        // out += bias[n]              (bias bf16, length N)
  MLF_EPI_GELU = 2,        // out = gelu_tanh(out)
  MLF_EPI_STORE_PRE = 4,   // aux_out[m,n] = value before the activation (bf16)
  MLF_EPI_RESIDUAL = 8,    // out += aux_in[m,n]          (bf16)
  MLF_EPI_DGELU_MUL = 16,  // out *= gelu_tanh'(aux_in[m,n])
  MLF_EPI_ACCUM = 32,      // out += previous contents of out
  MLF_EPI_OUT_FP32 = 64,   // out is fp32 instead of bf16
  MLF_EPI_SWIGLU = 128,    // columns come in (gate, up) pairs: out[m, n/2] = silu(gate) * up
  MLF_EPI_DSWIGLU = 256,   // aux_in holds (gate, up) pairs [M, 2N]; out[m, 2n..2n+1] = grads
};

// Optional in-kernel communication attached to a GEMM (all zero = plain GEMM).
typedef struct MlfGemmComm {
  // ---- gather side: one operand arrives in row chunks pulled from peers by copy CTAs ----
  int gather_operand;       // 0 none, 1 = A rows (M), 2 = B rows (N)
  int world;                // number of ranks W (<= 8)
  int rank;                 // this rank
  int n_copy_ctas;          // CTAs of the grid that copy instead of computing
  int rows_per_rank;        // operand rows owned by each rank (last rank may own fewer)
  int flag_rows;            // rows covered by one ready flag (multiple of the tile extent)
  int row_bytes;            // bytes per operand row in the peers' shards and the local buffer
  int _pad0;
  const void* src[8];       // src[r] = base of rank r's shard (peer-mapped)
  void* gathered;           // local full-size operand buffer the GEMM reads through TMA
  uint32_t* flags;          // [ceil(rows/flag_rows)] ready flags, zeroed before launch
  uint32_t* counters;       // same length, zeroed before launch
  // ---- scatter side: output rows are routed to their owner's partial buffer ----
  int scatter_out;          // 1 = route rows: out_peer[owner] + (rank*rows_per_owner + local_row)*ldo
  int rows_per_owner;       // output rows owned by each rank
  void* out_peer[8];        // out_peer[r] = rank r's partial buffer [W, rows_per_owner, ldo]
  // ---- piggy-backed copies: {src, dst, bytes} int64 triples (device array) the copy CTAs move
  //      after the gated chunks, with no ready flags (consumers are later kernels on the stream).
  //      May be used with gather_operand == 0 (n_copy_ctas must then still be set).
  const void* extra_segs;
  int n_extra;
  int _pad1;
} MlfGemmComm;

typedef struct MlfGemmArgs {
  const void* a;      // A: K-major [M, K] (a_mn = 0) or MN-major [K, M] (a_mn = 1), bf16
  const void* b;      // B: K-major [N, K] (b_mn = 0) or MN-major [K, N] (b_mn = 1), bf16
  void* out;          // [M, N] bf16 (or fp32 with MLF_EPI_OUT_FP32)
  const void* bias;   // bf16 [N] or null
  const void* aux_in; // bf16 [M, N] or null
  void* aux_out;      // bf16 [M, N] or null
  int M, N, K;
  int lda, ldb, ldo, ld_aux_in, ld_aux_out;  // row pitches in elements
  int a_mn, b_mn;
  int flags;
  float alpha;
  int tile_n;         // 0 = choose; else 64, 128 or 256
  int max_ctas;       // 0 = all SMs
  const MlfGemmComm* comm;  // host pointer or null
} MlfGemmArgs;

const char* mlf_last_error(void);
int mlf_read_status(int clear);
int mlf_sm_count(void);

int mlf_gemm_bf16(const MlfGemmArgs* args, uint64_t stream);

#ifdef __cplusplus
}
#endif
