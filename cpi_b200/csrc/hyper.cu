// Hyper-connections: a residual that is kept as S parallel streams x_1 .. x_S [S][tokens][width], float32.
//
// A sublayer reads one mixture of the streams and its output is spread over all of them:
//     u   = sum_s a[s] x_s                      (a: the sublayer's read weights)
//     y   = sublayer(norm(u))
//     x_t <- sum_s M[s][t] x_s + b[t] y         (M indexed [from][to], b: the write weights; all t from the old x)
// One kernel does both halves around a sublayer boundary, a block per token: it first applies the write-back of
// the sublayer that has just run (when `y` is given), then forms the next sublayer's u from the new streams and
// normalises it (when `h_out` is given), so the streams are read and written once per boundary.  With S = 1,
// a = b = M = 1 this is the ordinary residual sum followed by the next norm.
//
// The norm is x * rsqrt(mean(x^2) + eps) * (offset + w): offset 0 for a plain weight, 1 for a weight that is
// stored as its distance from one.  Sums are float32 in a fixed order per token, so a token's result does not
// depend on the other tokens of the launch.
#include "common.cuh"

namespace cpi {

constexpr int HC_MAX_STREAMS = 8;

struct HcParams {
  float* x; long stream_stride;          // [S][T][W] float32, stream_stride = T * W of the allocation
  int n_streams, width;
  const float* y; long y_stride;         // [T][W] float32 or null: no write-back
  const float* mix;                      // [S][S] from, to   (with y)
  const float* write;                    // [S]               (with y)
  const float* read;                     // [S] or null: every stream with weight one (with h_out)
  const int* rows;                       // token of output row r, or null: row r is token r (only without y)
  const void* norm_w; int norm_w_dtype; float norm_offset; float eps;
  void* h_out; long h_stride;            // [rows][W] in TO, or null: no norm
  float* sum_out;                        // [rows][W] float32 or null: also the plain mixture u (before the norm)
};

template <typename TO>
__global__ void __launch_bounds__(1024) hc_step_kernel(HcParams p) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float coef[HC_MAX_STREAMS * HC_MAX_STREAMS + 2 * HC_MAX_STREAMS];
  const int S = p.n_streams, W = p.width;
  float* mix_s = coef;
  float* write_s = coef + HC_MAX_STREAMS * HC_MAX_STREAMS;
  float* read_s = write_s + HC_MAX_STREAMS;
  // the coefficients are weights: no kernel writes them, so they are fetched before the wait
  if (threadIdx.x < S * S && p.y) mix_s[threadIdx.x] = p.mix[threadIdx.x];
  if (threadIdx.x < S) {
    if (p.y) write_s[threadIdx.x] = p.write[threadIdx.x];
    read_s[threadIdx.x] = p.read ? p.read[threadIdx.x] : 1.0f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const int t = p.rows ? p.rows[r] : r;
  float* xt = p.x + (size_t)t * W;
  const float* yt = p.y ? p.y + (size_t)t * p.y_stride : nullptr;
  constexpr int PER = 4;                                   // elements a thread keeps between the two passes
  float ss = 0.f;
  // write-back of the sublayer before (if any) and the mixture for the next one, at element i
  auto element = [&](int i) -> float {
    float xs[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s)
      if (s < S) xs[s] = xt[(size_t)s * p.stream_stride + i];
    if (yt) {
      const float yv = yt[i];
      float nx[HC_MAX_STREAMS];
#pragma unroll
      for (int to = 0; to < HC_MAX_STREAMS; ++to) {
        if (to < S) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) acc = fmaf(mix_s[s * S + to], xs[s], acc);
          nx[to] = fmaf(write_s[to], yv, acc);
        }
      }
#pragma unroll
      for (int s = 0; s < HC_MAX_STREAMS; ++s)
        if (s < S) { xs[s] = nx[s]; xt[(size_t)s * p.stream_stride + i] = nx[s]; }
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s)
      if (s < S) u = fmaf(read_s[s], xs[s], u);
    if (p.sum_out) p.sum_out[(size_t)r * W + i] = u;
    return u;
  };
  // The first PER elements of a thread: every load is issued before the first store (the streams are read and
  // written through one pointer, so the compiler would otherwise keep each element's loads behind the stores of
  // the one before: a round trip to memory per element).
  float u_keep[PER];
  {
    float xs[PER][HC_MAX_STREAMS], yv[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
#pragma unroll
      for (int s = 0; s < HC_MAX_STREAMS; ++s) xs[j][s] = (s < S && i < W) ? xt[(size_t)s * p.stream_stride + i] : 0.f;
      yv[j] = (yt && i < W) ? yt[i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      float u = 0.f;
      if (i < W) {
        if (yt) {
          float nx[HC_MAX_STREAMS];
#pragma unroll
          for (int to = 0; to < HC_MAX_STREAMS; ++to) {
            if (to < S) {
              float acc = 0.f;
#pragma unroll
              for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) acc = fmaf(mix_s[s * S + to], xs[j][s], acc);
              nx[to] = fmaf(write_s[to], yv[j], acc);
            }
          }
#pragma unroll
          for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) { xs[j][s] = nx[s]; xt[(size_t)s * p.stream_stride + i] = nx[s]; }
        }
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
          if (s < S) u = fmaf(read_s[s], xs[j][s], u);
        if (p.sum_out) p.sum_out[(size_t)r * W + i] = u;
      }
      u_keep[j] = u;
      ss = fmaf(u, u, ss);
    }
  }
  for (int i = threadIdx.x + PER * blockDim.x; i < W; i += blockDim.x) {     // a very wide row
    const float u = element(i);
    ss = fmaf(u, u, ss);
  }
  if (!p.h_out) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)W + p.eps);
  TO* o = reinterpret_cast<TO*>(p.h_out) + (size_t)r * p.h_stride;
  auto emit = [&](int i, float u) {
    float v = u * inv;
    if (p.norm_w) v *= p.norm_offset + load_any(p.norm_w, p.norm_w_dtype, i);
    o[i] = from_f32<TO>(v);
  };
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < W) emit(i, u_keep[j]);
  }
  for (int i = threadIdx.x + PER * blockDim.x; i < W; i += blockDim.x) {     // formed again from the new streams: same bits
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s)
      if (s < S) u = fmaf(read_s[s], xt[(size_t)s * p.stream_stride + i], u);
    emit(i, u);
  }
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_hc_step(float* x, long stream_stride, int n_streams, int n_rows, int width, const float* y,
                           long y_stride, const float* mix, const float* write, const float* read, const int* rows,
                           const void* norm_w, int norm_w_dtype, float norm_offset, float eps, void* h_out,
                           int h_dtype, long h_stride, float* sum_out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(n_streams >= 1 && n_streams <= HC_MAX_STREAMS, "hyper-connections: %d streams (supported: 1 to %d)",
              n_streams, HC_MAX_STREAMS);
  CPI_REQUIRE(width > 0, "hyper-connections: bad width %d", width);
  CPI_REQUIRE(!(y && rows), "hyper-connections: the write-back runs over all tokens, not over chosen rows");
  CPI_REQUIRE(!y || (mix && write), "hyper-connections: a write-back needs its mixing matrix and write weights");
  HcParams p{x, stream_stride, n_streams, width, y, y_stride, mix, write, read, rows,
             norm_w, norm_w_dtype, norm_offset, eps, h_out, h_stride, sum_out};
  // a thread takes four elements at most in one round of loads: wide rows get large blocks
  int threads = (width + 3) / 4;
  threads = threads <= 64 ? 64 : (threads <= 128 ? 128 : (threads <= 256 ? 256 : (threads <= 512 ? 512 : 1024)));
  CPI_DISPATCH_DTYPE(h_dtype, TO, cpi::launch_pdl(hc_step_kernel<TO>, n_rows, threads, 0, stream, p));
  return check_launch("hc_step");
}
