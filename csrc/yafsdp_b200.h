// C interface of the native sm_100a library (libyafsdp_b200.so).  Every function launches on the
// given CUDA stream (a cudaStream_t passed as void*) and returns 0 on success, a negative value on
// a rejected argument (-1), a tensor-map failure (-2) or a CUDA error (-cudaError_t).  Nothing here
// synchronises the device.  Python binds these symbols through ctypes.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int yf_version(void);
int yf_sm_count(void);
// First error recorded by any kernel of the library, on any GPU of this process, since the last clearing read (0 = none).
// The status word sits in host memory: the call neither synchronises nor touches a GPU, so it is cheap enough to poll
// every step.  It reports what kernels have written so far; synchronise first to cover work still in flight.
int yf_status_read(int* code, int* site, int clear);

// ---- tcgen05 GEMM family (gemm.cu)
int yf_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, float alpha, int sm_limit, void* stream);

int yf_gemm_bf16_sumsq(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, float alpha, int sm_limit, float* sumsq,
                       void* stream);
/* C = alpha * A * B^T + R: bf16 output, bf16 residual R [M,N] (row pitch ldr) added in fp32 in the epilogue; C may be R. */
int yf_gemm_bf16_residual(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, long long ldr, int a_mn, int b_mn, float alpha, int sm_limit, void* stream);
// fused all-gather -> GEMM and GEMM -> reduce-scatter (same kernel, see gemm.cu for the argument contracts)
int yf_gemm_bf16_gathered(const void* A, void* C, int M, int N, int K, long long lda, long long ldc, int a_mn, int out_f32,
                          void* const* peer_in, void* layer_buf, long long shard_bytes, long long b_byte_off, int rank, int world,
                          void* counters, long long epoch, void* stream);
int yf_gemm_bf16_scatter(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int a_mn, int b_mn,
                         float alpha, void* const* peer_grad, long long c_flat_off, long long shard_numel, int rank, int world,
                         int wire_bf16, int sm_limit, void* stream);

// grouped GEMM -> reduce-scatter: the weight-gradient GEMMs of a layer (n <= 4 problems sharing K and the operand majors, in
// ascending order of flat_off) as one launch that deals the owners' tiles round-robin (see gemm.cu)
int yf_gemm_bf16_scatter_grouped(int n, const void* const* A, const void* const* B, const int* M, const int* N, int K,
                                 const long long* lda, const long long* ldb, int a_mn, int b_mn, float alpha, void* const* peer_grad,
                                 const long long* flat_off, long long shard_numel, int rank, int world, int wire_bf16, int sm_limit,
                                 void* stream);

// ---- memory-bound kernels (elementwise.cu)
int yf_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int D, float eps, void* stream);
/* dx (+ dres) and dw += column sums of dy * xhat; zero_dw: dw is cleared first, inside the dx kernel (no fill launch) */
int yf_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                   float* dw, int zero_dw, int T, int D, void* stream);
int yf_rope(void* qkv, const float* cos_sin, int T, int seq_len, long long row_stride, int col0, int n_heads,
            int head_dim, int backward, void* stream);
int yf_swiglu_fwd(const void* gu, void* h, long long T, int F, void* stream);
int yf_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long T, int F, void* stream);
int yf_cross_entropy(void* logits, const long long* labels, float* loss_rows, int T, int V, long long ldl,
                     float grad_scale, const float* scale_ptr, int write_grad, void* stream);
int yf_embedding_fwd(const void* table, const long long* ids, void* out, long long T, int D, int V, void* stream);
int yf_embedding_bwd(const void* dout, const long long* ids, float* dtable, long long T, int D, int V, void* stream);
int yf_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, const float* grad_scale_ptr, long long n,
             float lr, float beta1, float beta2, float eps, float weight_decay, int step, int max_ctas, void* stream);
int yf_sumsq(const float* g, long long n, float* out, void* stream);
int yf_clip_coef(const float* total_sq, float max_norm, float* coef, float* norm_out, void* stream);
int yf_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream);
int yf_accum_bf16_to_f32(const void* src, float* dst, long long n, float scale, int accumulate, void* stream);
int yf_add_bf16(const void* a, const void* b, void* y, long long n, void* stream);

// ---- flash attention, head_dim 128 (attn_fwd.cu, attn_bwd.cu)
int yf_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Hq, int Hkv,
                long long q_stride, long long kv_stride, long long out_stride, float scale, int causal, void* stream);
int yf_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                float* delta, float* dq_accum, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                long long q_stride, long long kv_stride, long long o_stride, long long do_stride, long long dq_stride,
                long long dkv_stride, float scale, int causal, void* stream);

// No counterpart in the reference.  yf_attn_bwd for callers that cannot allocate device memory (a plain C host
// without a tensor framework, or a job whose own pool already holds the whole GPU): the delta / dQ-accumulator
// scratch is a fixed device array inside the library (about 16.1 MiB per GPU, held until exit), so the call takes
// no scratch arguments and never calls cudaMalloc / cudaFree or an allocating library routine.  Refuses B*S*Hq > 32768
// with -3.  The first call on a device resolves the array's address: make it before any stream capture.  Calls
// on one device share the array (the part that must be zero is cleared each call); calls that overlap on the GPU race.
int yf_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                        void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, long long q_stride, long long kv_stride,
                        long long o_stride, long long do_stride, long long dq_stride, long long dkv_stride, float scale,
                        int causal, void* stream);

// ---- peer-memory collectives over NVLink (comm.cu); peer arrays are host arrays of `world` device pointers
int yf_allgather_pull(void* const* peer_in, void* out, long long shard_bytes, int rank, int world, int n_ctas, void* stream);
int yf_reduce_scatter_pull(void* const* peer_in, float* dst, long long shard_numel, int rank, int world, float scale,
                           int accumulate, int bf16_wire, int n_ctas, void* stream);
int yf_reduce_scatter_pull_sumsq(void* const* peer_in, float* dst, long long shard_numel, int rank, int world, float scale,
                                 int accumulate, int bf16_wire, int n_ctas, float* sumsq, void* stream);
int yf_reduce_scatter_mc(const void* mc_in, float* dst, long long shard_numel, int rank, int world, float scale, int accumulate,
                         int bf16_wire, int n_ctas, float* sumsq, void* stream);
int yf_allgather_mc(const void* in, void* mc_out, long long shard_bytes, int rank, int world, int n_ctas, void* stream);
// Push fp32 values of the flat layer gradient into the owners' reduce-scatter slots (companion of yf_gemm_bf16_scatter for
// gradients that no GEMM produces); src may be null (zeros).  numel, flat_off and shard_numel must be multiples of 4 (8 with
// the bf16 wire format, where the values are rounded to bf16 on the way).
int yf_push_flat(const float* src, long long numel, long long flat_off, void* const* peer_grad, long long shard_numel, int rank,
                 int world, int wire_bf16, void* stream);
// Signal pads (sequence-numbered flags in every rank's peer-mapped pad): mode 1 = raise this rank's word of `slot` to `seq`
// in every pad, mode 2 = wait (bounded) until every rank's word of `slot` in the own pad has reached `seq`, 3 = both.
int yf_signal_pad(void* const* pads, int rank, int world, int slot, long long seq, long long timeout_ms, int mode, void* stream);
int yf_signal_barrier(void* const* pads, int rank, int world, int slot, long long seq, long long timeout_ms, void* stream);
int yf_flag_wait(const void* flags, long long index, long long value, long long timeout_ms, void* stream);
int yf_flag_set(void* flags, long long index, long long value, void* stream);
int yf_memcpy_async(void* dst, const void* src, long long nbytes, void* stream);
int yf_ipc_alloc(long long nbytes, void** ptr_out, void* handle_out64);
int yf_ipc_open(const void* handle64, void** ptr_out);
int yf_ipc_close(void* ptr);
int yf_ipc_free(void* ptr);

#ifdef __cplusplus
}
#endif
