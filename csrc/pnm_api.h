// C ABI of the sm_100a kernel library (libpnm_b200.so).  All pointers are device pointers
// unless stated otherwise; `stream` is a cudaStream_t.  Every function returns 0 on success
// and a negative code when an argument is rejected or a launch fails.  Device-side
// time-outs of bounded waits are reported through pnm_get_error().
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int pnm_version();
int pnm_num_sms();
int pnm_get_error();    // synchronising read of the device error word (0 = none)
int pnm_reset_error();

// C[M,N] = epilogue(A[M,K] * B[N,K]^T); bf16 in/out, fp32 accumulate.  See gemm_tn.cuh.
int pnm_gemm_tn(const void* A, int lda, const void* A2, int lda2, const void* A3, int lda3, const void* B, int ldb, void* C, int ldc, void* Z,
                int ldz, const void* AUX, int ldaux, int M, int N, int K, int K1, int K2, const float* bias,
                const float* scale, float* group_out, int act, int aux_mode, int scale_post, int bn, int max_ctas,
                void* stream);

// out[Na,Nb] (fp32) += A[M,Na]^T * B[M,Nb];  colsum[Na] += column sums of A (optional).
int pnm_gemm_nt(const void* A, int lda, const void* B, int ldb, float* out, int ldo, float* colsum, int M, int Na,
                int Nb, int max_ctas, void* stream);
// Stacked batches of equal problems in one launch (rows of a problem padded to Mp; see pnm_lib.cu)
int pnm_gemm_tn_stacked(const void* A, int lda, const void* B, int ldb, void* C, int ldc, const void* AUX, int ldaux, int Mp, int N,
                        int K, int batch, const float* bias, int act, int aux_mode, int max_ctas, void* stream);
int pnm_gemm_nt_stacked(const void* A, int lda, const void* B, int ldb, float* out, float* colsum, int Mp, int Na, int Nb, int batch,
                        int max_ctas, void* stream);

// y = LN(x [+ r]) [+ post]; bf16 rows of C channels (C % 8 == 0, C <= 1024), fp32 gamma / beta / statistics.
int pnm_layernorm_fwd(const void* x, const void* r, const float* gamma, const float* beta, void* y, void* sum_out,
                      float* mean, float* rstd, const void* post, long long M, int C, float eps, void* stream);
long long pnm_layernorm_bwd_scratch_floats(long long M, int C);
int pnm_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                      const void* dres, void* dx, float* dgamma, float* dbeta, float* scratch, long long M, int C,
                      void* stream);

// out[e,:] = in[idx[e],:] (* scale[idx[e]]); bf16 rows, int32 indices (idx may be null = identity).
int pnm_gather_rows(const void* in, int ldi, const int* idx, const float* scale, void* out, int ldo, long long E,
                    int C, void* stream);
// out[n,:] (+)= sum over k in [offsets[n], offsets[n+1]) of in[perm[k],:]; mode 1 divides by the count.
int pnm_segment_sum(const void* in, int ldi, const int* perm, const int* offsets, void* out, int ldo, long long N,
                    int C, int accumulate, int mode, void* stream);

// In-kernel all-reduce (sum, fp32) over peer-mapped symmetric buffers; see peer.cuh for the layout.
// bases: host array of `world` peer-mapped base pointers; epoch_base: optional device uint32 added to epoch (lets a
// captured CUDA graph advance the call numbers on replay); max_ctas: 0 = default.  On a time-out the outputs are NaN.
int pnm_peer_allreduce(const float* in, float* out, long long n, float scale, int two_shot, const void* const* bases,
                       int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s,
                       void* stream, const void* epoch_base, int max_ctas);
// Gradient-bucket all-reduce, bf16 on the wire: io[i] <- sum over ranks of bf16(scale * io[i]) (fp32 accumulation), in place;
// cast, reduce-scatter and all-gather are one kernel.  n % 8 == 0, io 32-byte aligned, n <= 2 * capacity_floats.
int pnm_peer_allreduce_bf16(float* io, long long n, float scale, const void* const* bases, int rank, int world,
                            unsigned int epoch, long long capacity_floats, double budget_s, void* stream,
                            const void* epoch_base, int max_ctas);
// Building blocks of staged transfers.  pnm_peer_signal raises this rank's flag of call `epoch` on every peer (data written
// before it on the stream is then readable); pnm_peer_pull copies `bytes` from a peer-mapped address into local memory after
// rank flag_from's flag arrived (flag_from < 0: no wait); pnm_peer_pull_reduce sums block [rank * block, (rank + 1) * block) of
// every rank's stage A into dst after all flags arrived (reduce-scatter in the pull model).
int pnm_peer_signal(const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                    void* stream, const void* epoch_base);
int pnm_peer_pull(const void* src, void* dst, long long bytes, int flag_from, const void* const* bases, int rank, int world,
                  unsigned int epoch, long long capacity_floats, double budget_s, void* stream, const void* epoch_base,
                  int max_ctas);
int pnm_peer_pull_reduce(float* dst, long long block, const void* const* bases, int rank, int world, unsigned int epoch,
                         long long capacity_floats, double budget_s, void* stream, const void* epoch_base, int max_ctas);
int pnm_peer_sum_blocks(float* dst, const void* const* srcs, long long n, int wait, const void* const* bases, int rank, int world,
                        unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream,
                        int max_ctas);
// Row softmax over bf16 rows (softmax_rows.cu): forward in place with optional log-sum-exp, backward over dP in place.
int pnm_softmax_rows_fwd(void* S, long long ld, long long rows, int L, float scale, float* lse, void* stream);
int pnm_softmax_rows_bwd(const void* P, long long ldp, void* dP, long long ldd, long long rows, int L, float scale, void* stream);
// Enqueue a copy of the device error word into pinned host memory (non-blocking poll of the bounded waits).
int pnm_error_copy_async(int* pinned_host, void* stream);
int pnm_peer_flag_bytes();
int pnm_peer_wait_probe(const void* flag, unsigned int expect, double budget_s, int* status_out, void* stream);

// Multi-tensor Adam / AdamW over a device table of tensors (layout in optim.cu); fp32 parameters and moments.
int pnm_opt_chunk();
int pnm_adam_multi(const void* entries, const void* blocks, int n_blocks, float lr, float b1, float b2, float eps,
                   float wd, float step_size, float inv_bc2_sqrt, int decoupled, float grad_scale, void* stream,
                   const float* hyper);  // hyper: optional device {lr, step}; overrides lr / step_size / inv_bc2_sqrt
int pnm_grad_sqnorm_multi(const void* entries, const void* blocks, int n_blocks, float* out, void* stream);

// Periodic stencil programs (layout in stencil.cu): gradients, divergence, curl, Laplacians and their transposes.
int pnm_stencil_max_terms();
int pnm_stencil_program_bytes();
int pnm_stencil_apply(const void* in, void* out, const void* tables, const void* prog_host, int dtype, void* stream);

// Mesh gradient reconstruction (mesh_grad.cu). backward != 0 runs the transposed pass for the values
// (vals = upstream gradient [n, D, C], out = dvals [n, C], zero-initialised by the caller).
int pnm_mesh_lsq_gradient(const float* pts, const float* vals, const long long* offs, const long long* nbr, float* out,
                          long long n, int D, int C, float weight_power, float eps, int min_neighbors, int backward,
                          void* stream);
int pnm_mesh_green_gauss(const float* a, const long long* idx, const float* vals, float* out, long long n_cells, int D,
                         int C, int mode, void* stream);

// Grid <-> point interpolation (interp.cu): gather (scatter == 0) or atomic scatter of point values onto the grid.
int pnm_interp(const float* pts, const float* src, float* dst, const float* grid_desc, const int* n, int dims, int type,
               long long npts, int C, int scatter, void* stream);

// Neighbour queries (neighbors.cu). Points are pre-sorted by cell of a uniform grid; `order` maps sorted -> original.
int pnm_radius_count(const float* pts_sorted, const int* cell_start, const int* cell_end, const float* queries,
                     int* counts, const float* lo, float cell, const int* n, int nq, float radius, void* stream);
int pnm_radius_fill(const float* pts_sorted, const int* order, const int* cell_start, const int* cell_end,
                    const float* queries, const long long* offsets, long long* pairs, long long total, const float* lo,
                    float cell, const int* n, int nq, float radius, void* stream);
int pnm_radius_topk(const float* pts_sorted, const int* order, const int* cell_start, const int* cell_end,
                    const float* queries, long long* idx, float* d2, const float* lo, float cell, const int* n, int nq,
                    int K, float radius, void* stream);
int pnm_knn_max_k();
int pnm_knn(const float* pts, const float* queries, long long* idx, float* dist, int np, int nq, int D, int K, void* stream);
// Farthest point sampling, one CTA per cloud; scratch: [B, N] floats; out: [B, S] int64, column 0 preset to the first sample.
int pnm_fps(const float* pts, float* scratch, long long* out, int B, int N, int S, void* stream);

// PDE data generators (pde_darcy.cu, pde_kh.cu): each solve / simulation is one cooperative launch.
int pnm_darcy_permeability(const float* fourier, float* perm, int B, int res, int nf, float kmin, float kmax, void* stream);
int pnm_darcy_solve(float* u0, float* u1, const float* perm, unsigned int* residual, int B, int res, int levels,
                    int max_iterations, int check_every, float threshold, void* stream);
int pnm_kh_simulate(float* cons, float* faces, const float* w, float* snap_rho, float* snap_vel, float* snap_p, int B, int N,
                    int nfreq, int snapshots, int steps_per_snapshot, float gamma, float dx, float dt, float sigma, void* stream);

// Triangle-mesh queries over an implicit BVH (bvh.cu): bounds [2L-1, 2, 3], order [L] (triangle per leaf, -1 = padding),
// tris [F, 3, 3]. Misses: NaN distance / point and face -1 (closest), inf distance and face -1 (ray cast).
int pnm_bvh_closest(const float* bounds, const int* order, const float* tris, const float* queries, float* out_dist,
                    float* out_point, long long* out_face, int n_leaves, long long nq, float max_dist, void* stream);
int pnm_bvh_raycast(const float* bounds, const int* order, const float* tris, const float* origins, const float* dirs,
                    float* out_t, long long* out_face, float* out_uv, int n_leaves, long long nr, float max_distance,
                    void* stream);
int pnm_winding_number(const float* tris, const float* queries, float* out, long long n_tris, long long nq, void* stream);

// Headless renderers (render.cu). camera = {eye, forward, right, up} as 12 floats; bounds = {min xyz, max xyz};
// RGBA volumes / colour fields are channels-last float4; outputs rgba [H*W*4], depth [H*W] (3.4e38 = nothing hit),
// normal [H*W*3].  The splatting renderers need winners [H*W] pre-filled with empty_key.
int pnm_volume_render(const float* vol, const float* camera, const float* bounds, int W, int H, float step, int max_steps,
                      float tan_half, float aspect, float opacity_stop, float depth_thr, int nx, int ny, int nz, float* rgba,
                      float* depth, void* stream);
int pnm_isosurface_render(const float* field, const float* color_field, const float* camera, const float* bounds,
                          const float* uniform_color, const float* light, int W, int H, float threshold, float step,
                          int max_steps, float tan_half, float aspect, float ambient, int has_color_field, int nx, int ny,
                          int nz, float* rgba, float* depth, float* normal, void* stream);
int pnm_mesh_raycast_render(const float* bvh_bounds, const int* order, const float* tris, const int* indices, int n_leaves,
                            const float* colors, const float* camera, const float* uniform_color, const float* light, int W,
                            int H, float tan_half, float aspect, float max_distance, float ambient, int color_mode,
                            float* rgba, float* depth, float* normal, void* stream);
int pnm_point_cloud_render(const float* points, const float* colors, const float* camera, const float* uniform_color, int W,
                           int H, float tan_half, float aspect, float z_near, float z_far, int point_size, long long n,
                           float depth_scale, long long empty_key, int has_colors, long long* winners, float* rgba,
                           float* depth, void* stream);
int pnm_wireframe_render(const float* edges, const float* camera, const float* uniform_color, int W, int H, float tan_half,
                         float aspect, float z_near, float z_far, int thickness, long long n, float depth_scale,
                         long long empty_key, long long* winners, float* rgba, float* depth, void* stream);
int pnm_line_integral_convolution(const float* vec, const float* seed, float step, int num_steps, float contrast, int nx,
                                  int ny, int nz, float* out, void* stream);
int pnm_scalar_field_to_rgba(const float* field, long long n, float vmin, float vmax, float max_opacity,
                             float opacity_threshold, unsigned char* out, void* stream);
int pnm_vector_field_to_rgba(const float* vec, const float* lic, long long n, float vmin, float vmax, float max_opacity,
                             float lic_threshold, unsigned char* out, void* stream);

// GroupNorm (+ fused SiLU) forward / backward (groupnorm.cu).  dtype: 0 bf16, 1 fp32; layout: 0 channels-first,
// 1 channels-last; act: 0 none, 1 SiLU; S = number of spatial slices; scratch holds pnm_groupnorm_scratch_floats floats.
// Return value -1: shape not covered by these kernels.  dgamma / dbeta must be zeroed by the caller.
long long pnm_groupnorm_scratch_floats(int B, int C, int G, int S);
int pnm_groupnorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, float* scratch,
                      int B, int C, long long HW, int G, int S, int layout, int dtype, int act, float eps, void* stream);
int pnm_groupnorm_bwd(const void* x, const void* dy, const float* gamma, const float* beta, const float* mean,
                      const float* rstd, void* dx, float* dgamma, float* dbeta, float* scratch, int B, int C, long long HW,
                      int G, int S, int layout, int dtype, int act, void* stream);

// GroupNorm over a row-sharded channels-last image: moments over all ranks' rows, summed inside the normalising kernel by
// peer loads (see groupnorm.cu).  hw_global = pixels per image of the whole image; counter = zeroed device uint32.
int pnm_groupnorm_fwd_sharded(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                              float* scratch, int B, int C, long long HW, long long hw_global, int G, int S, int dtype, int act,
                              float eps, const void* const* bases, int rank, int world, unsigned int epoch,
                              long long capacity_floats, double budget_s, const void* epoch_base, void* counter, void* stream);
int pnm_groupnorm_bwd_sharded(const void* x, const void* dy, const float* gamma, const float* beta, const float* mean,
                              const float* rstd, void* dx, float* dgamma, float* dbeta, float* scratch, int B, int C,
                              long long HW, long long hw_global, int G, int S, int dtype, int act, const void* const* bases,
                              int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s,
                              const void* epoch_base, void* counter, void* stream);

// out = silu^(order)(x) * g (g may be null), order 0..4; dtype 0 bf16, 1 fp32; pointers 16-byte aligned (-2 otherwise).
int pnm_silu_derivative(const void* x, const void* g, void* out, long long n, int order, int dtype, void* stream);

// Neighbourhood attention over [B, L, H, D] tensors, L = prod(shape[0..nd)) (natten.cu).  dtype 0 bf16, 1 fp32.
// Returns -1 when the geometry is outside the kernels' limits (<= 512 neighbours, D <= 256).
int pnm_natten_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int D, int nd, const int* shape,
                   const int* kernel, const int* dilation, float scale, int dtype, void* stream);
int pnm_natten_bwd(const void* q, const void* k, const void* v, const void* dout, void* dq, float* dk, float* dv, int B, int H,
                   int D, int nd, const int* shape, const int* kernel, const int* dilation, float scale, int dtype,
                   void* stream);

// Stride-1 "same" 2-D convolution of a channels-last bf16 image as an implicit GEMM on the tensor cores (gemm_tn.cuh):
// x [n, h, w, cin], weight [cout, ksize*ksize*cin] (tap-major), y [n, h, w, cout]; bias fp32 [cout] or null;
// act as in pnm_gemm_tn.  cin % 64 == 0, cout % 8 == 0, odd ksize <= 7.
int pnm_conv2d_nhwc(const void* x, const void* weight, void* y, int n, int h, int w, int cin, int cout, int ksize,
                    const float* bias, int act, int bn, int max_ctas, void* stream);

// Halo exchange fused into the 3 x 3 convolution of a height-sharded image (gemm_tn.cuh, conv mode with halo):
// pnm_halo_publish copies this slab's first / last rows into its mailbox and raises the neighbours' flags;
// pnm_conv2d_nhwc_halo reads the neighbours' rows (peer-mapped) inside the convolution kernel once their flags carry
// `epoch`; interior tiles are computed first.  Null row / flag pointers mark the outer edges (zero padding).
int pnm_halo_publish(const void* x, void* top, void* bottom, int n, int h, int w, int c, void* flag_at_up, void* flag_at_down,
                     unsigned int epoch, void* counter, void* stream);
int pnm_conv2d_nhwc_halo(const void* x, const void* weight, void* y, int n, int h, int w, int cin, int cout, const float* bias,
                         int act, const void* up_rows, const void* down_rows, const void* flag_up, const void* flag_down,
                         unsigned int epoch, int bn, int max_ctas, void* stream, double budget_s);  // budget_s 0 = default (2 s)
// Weight (and bias) gradient of the 3 x 3 stride-1 "same" convolution as a split reduction over pixel patches on the tensor
// cores (gemm_nt.cuh, conv mode): out [cout, 9 * cin] fp32 tap-major and colsum [cout] are ACCUMULATED into.  up_rows /
// down_rows: input rows just above / below a height slab (local copies or peer-mapped); with flag_up / flag_down the kernel
// waits until they carry `epoch`.  cin % 64 == 0, cout % 8 == 0, cout >= 64; with halo rows h % 4 == 0.
int pnm_conv2d_wgrad_nhwc(const void* dy, const void* x, float* out, float* colsum, int n, int h, int w, int cin, int cout,
                          const void* up_rows, const void* down_rows, const void* flag_up, const void* flag_down,
                          unsigned int epoch, double budget_s, int max_ctas, void* stream);

// out[BH,Sq,D] = softmax(scale * q k^T (+ causal mask, top-left aligned)) v for contiguous bf16 q [BH,Sq,D], k [BH,Skv,D] and
// v [BH,Skv,D] (v_transposed = 0) or v^T [BH,D,ldv] with ldv >= Skv, ldv % 8 == 0 (v_transposed = 1); D in {64, 128};
// lse [BH,Sq] (fp32, optional) receives the natural-log sum of exponentials of every row; p_in_tmem = 1 keeps the probability
// tile in tensor memory as the A operand of the second MMA instead of staging it in shared memory.  See flash_attn.cuh.
int pnm_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int BH, int Sq, int Skv, int D,
                       int ldv, float scale, int causal, int v_transposed, int p_in_tmem, void* stream);

// EDM noise conditioning: out[B,E] (fp32) = silu(W1 silu(W0 (emb + extra) + b0) + b1) with emb[b] = [sin(noise[b] f), cos(noise[b] f)],
// f = freqs[C/2]; extra [B,C] fp32 optional; weights row-major [E,C] and [E,E], biases optional; weight_dtype 0 = bf16, 1 = fp32.
int pnm_edm_conditioning(const float* noise, const float* freqs, const float* extra, const void* w0, const void* b0, const void* w1,
                         const void* b1, float* out, int B, int C, int E, int weight_dtype, void* stream);

// out[p,q,m] (+)= sum_r A[p,r,m] * B[r,q,m] over complex64 tensors; m = block of nd <= 4 mode dimensions (extents `shape`, complex-element
// strides sa / sb / so per tensor); chan_strides = {A_p, A_r, B_r, B_q, out_p, out_q}.  See spectral.cu.
int pnm_spectral_contract(const void* A, const void* B, void* out, int nd, const int* shape, const long long* sa, const long long* sb,
                          const long long* so, const long long* chan_strides, int P, int Q, int R, int conj_a, int conj_b,
                          int accumulate, void* stream);

// Equivariant normalisation of spherical-harmonic grids x[B, L, M, 2, C] (see sh_norm.cu): degree groups `group[L]`, statistic weights
// wstat[L, M], affine a[L, C], optional bias[C] on the (0, 0, 0) row, mask[L, M, 2].  dtype 0 = fp32, 1 = bf16, 2 = fp16.
int pnm_sh_norm_fits(int L, int M, int C, int which);
int pnm_sh_norm_bwd_grid(long long B, int L, int M, int C);
int pnm_sh_norm_fwd(const void* x, void* y, const float* aw, const float* bias, const float* wstat, const float* mask, const int* group,
                    long long B, int L, int M, int C, float eps, int subtract_mean, int dtype, void* stream);
int pnm_sh_norm_bwd(const void* x, const void* dy, void* dx, const float* aw, const float* wstat, const float* mask, const int* group,
                    float* daw_part, float* dbias_part, long long B, int L, int M, int C, float eps, int subtract_mean, int dtype,
                    int grid, void* stream);

// Pixel / observation cross attention in token space and the counting sort that packs observations by pixel (see pixel_attn.cu).
int pnm_pixel_attn_fwd(const void* qk, const void* tok, const int* cu, void* ctx, float* lse, int P, int H, int Dt, int dtype, void* stream);
int pnm_pixel_attn_bwd(const void* qk, const void* tok, const int* cu, const void* dctx, const float* lse, const float* delta, float* dqk,
                       float* dtok, int P, int H, int Dt, long long N, int atomic, int dtype, void* stream);
int pnm_counting_histogram(const int* idx, int* counts, long long n, int bins, int* bad, void* stream);
int pnm_counting_scatter(const int* idx, const int* offsets, int* cursor, int* order, long long n, int bins, void* stream);

// 2 x 2 box resampling of a channels-last bf16 image (mode 0: down, sum of the four pixels times scale; mode 1: up,
// replication times scale); c % 8 == 0
int pnm_resample2x_nhwc(const void* x, void* y, int n, int h, int w, int c, int mode, float scale, void* stream);

// Physics-attention small algebra (csrc/physics_attn_small.cu), partitioned-graph halo exchange (csrc/graph_halo.cu) and the
// AFNO spectral filter (csrc/afno_spectral.cu); argument conventions are documented above each definition.
int pnm_pa_prepare_fwd(const float* Wx, const float* bx, const float* Wfx, const float* Ws, const float* bs, const float* temp, void* Wc16, float* bc, float* inv_t, void* Wfx16, void* Wback16, int H, int D, int C, void* stream);
int pnm_pa_tokens_fwd(const void* const* srcs, int world, int use_flags, long long norm_off, int ld_tok, const float* Wqkv, const float* Wo, void* wcomb16, void* const* saved, int H, int D, int Cout, float scale, const void* const* bases, int rank, unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream);
int pnm_pa_tokens_bwd(const void* const* srcs, int world, int use_flags, const float* Wqkv, const float* Wo, void* const* saved, float* dWo, float* dWqkv, float* d_norm, void* Bcat16, void* BdT16, int H, int D, int Cout, float scale, float share, const void* const* bases, int rank, unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream);
int pnm_pa_prepare_bwd(const float* dWc, const float* dbc, const float* grp, const float* Wx, const float* bx, const float* Ws, const float* temp, float* dWx, float* dbx, float* dWs, float* dbs, float* dtemp, int H, int D, int C, void* stream);
int pnm_graph_halo_publish(const void* in, int ldi, const int* send_idx, void* mailbox, long long n_send, int C, const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats, const void* epoch_base, void* counter, void* stream);
int pnm_graph_gather_halo(const void* in, int ldi, const int* idx, int n_local, const int* halo_owner, const int* halo_slot, const void* const* mailboxes, void* out, int ldo, long long E, int C, int wait, const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream);
int pnm_graph_halo_pull_add(void* dn, int ldn, const int* bnd_row, const int* bnd_off, const int* ent_peer, const int* ent_slot, const void* const* mailboxes, long long n_bnd, int C, int wait, const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream);
int pnm_afno_rows_r2c(const void* const* tokens, void* Y, const int* geom, long long Tp, int kweight, int wait, const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream);
int pnm_afno_rows_c2r(const void* X, const void* const* tokens, const int* geom, long long Tp, int kweight, int signal, const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats, const void* epoch_base, void* counter, void* stream);
int pnm_afno_cols_fwd(const void* Y, void* Yout, void* Zs, void* O1s, void* O2s, const float* w1, const float* b1, const float* w2, const float* b2, int nb, const int* geom, float lambda, void* stream);
int pnm_afno_cols_bwd(const void* dYout, void* dY, const void* Zs, const void* O1s, const void* O2s, const float* w1, const float* w2, float* dw1, float* db1, float* dw2, float* db2, int nb, const int* geom, void* stream);
int pnm_afno_cols_dft(const void* Y, void* E, const void* mask, const int* geom, int Mp, float lambda, void* stream);
int pnm_afno_rows_c2r_add(const void* X, void* out, const void* add0, const void* add1, const int* geom, long long Tp, int kweight,
                          void* stream);
int pnm_afno_cols_idft(const void* E, void* Yout, const int* geom, int Mp, float lambda, void* stream);

// out = (a + b) * scale over n bf16 elements (n % 8 == 0; b may be null)
int pnm_add_scale_bf16(const void* a, const void* b, void* out, long long n, float scale, void* stream);

// Tokens [B, h, w, p0 * p1 * C] (features ordered (i, j, c)) <-> image [B, C, h * p0, w * p1], bf16.  to_image = 1 writes
// the image from the tokens, 0 writes the tokens from the image.  Returns -2 for shapes the kernel does not cover.
int pnm_unpatchify_bf16(void* tokens, void* image, int B, int h, int w, int p0, int p1, int C, int to_image, void* stream);

// out[0] = scale * sum((pred - tgt)^2) over n elements; dtype codes 0 = fp32, 1 = bf16; partial holds
// pnm_sq_err_partials() floats.  pnm_sq_err_grad writes grad = coef * gout[0] * (pred - tgt) in pred's dtype.
int pnm_sq_err_partials(void);
int pnm_sq_err_sum(const void* pred, const void* tgt, long long n, int pred_dtype, int tgt_dtype, double scale, float* partial,
                   float* out, void* stream);
int pnm_sq_err_grad(const void* pred, const void* tgt, const float* gout, long long n, int pred_dtype, int tgt_dtype, float coef,
                    void* grad, void* stream);

// Metadata features of observations (see obs_features.cu): out [n, 28] (extended = 0) or [n, 30] (extended = 1), fp32.
// lat is read only in the extended scheme; time_ns / target_s are int64 nanoseconds / seconds since the epoch.
int pnm_obs_metadata(const float* lat, const float* lon, const long long* time_ns, const long long* target_s, const float* height,
                     const float* pressure, const float* scan, const float* sat_zen, const float* sol_zen, float* out, long long n,
                     int extended, void* stream);

#ifdef __cplusplus
}
#endif
