// Vision preprocessing in one pass: bilinear resample of the source into its letterbox, mid-grey padding,
// normalisation (x/255 - 0.5)/0.5 and patch extraction to the ViT's input layout; plus the 2-D rotary of the
// tower and the 3x3 unfold of the aligner.  Reference behaviour: kernels/opt_vision_sm121.cu,
// crates/sparkflash-vision/src/{resample,prep}.rs; docs/architecture/06-vision.md sections 2-4.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sfb {

// one thread per output element; out[(py * nvw + px)][c * P * P + iy * P + ix]
__global__ void vision_prepare_kernel(const uint8_t* __restrict__ img, int W, int H, int x0, int y0, int w, int h, int dw, int dh,
                                      int P, int grey, __nv_bfloat16* __restrict__ out) {
  const int nvw = dw / P;
  const long long total = (long long)dw * dh * 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row_len = 3 * P * P;
    const long long patch = i / row_len;
    const int r = (int)(i % row_len);
    const int c = r / (P * P), iy = (r / P) % P, ix = r % P;
    const int y = (int)(patch / nvw) * P + iy, x = (int)(patch % nvw) * P + ix;
    float v = (float)grey;
    if (x >= x0 && x < x0 + w && y >= y0 && y < y0 + h) {
      float sy = ((y - y0) + 0.5f) * ((float)H / h) - 0.5f;
      float sx = ((x - x0) + 0.5f) * ((float)W / w) - 0.5f;
      sy = fminf(fmaxf(sy, 0.f), (float)(H - 1)); sx = fminf(fmaxf(sx, 0.f), (float)(W - 1));
      const int yi = (int)floorf(sy), xi = (int)floorf(sx);
      const int yj = min(yi + 1, H - 1), xj = min(xi + 1, W - 1);
      const float fy = sy - yi, fx = sx - xi;
      const float a = img[((size_t)yi * W + xi) * 3 + c], b = img[((size_t)yi * W + xj) * 3 + c];
      const float d = img[((size_t)yj * W + xi) * 3 + c], e = img[((size_t)yj * W + xj) * 3 + c];
      const float top = a * (1.f - fx) + b * fx, bot = d * (1.f - fx) + e * fx;
      v = top * (1.f - fy) + bot * fy;
    }
    out[i] = __float2bfloat16((v / 255.0f - 0.5f) / 0.5f);
  }
}

// half-split rotary over the whole head: pairs (k, k + hd/2); even frequency index uses the row position,
// odd the column position.  x: [N, heads, hd] bf16, in place.
__global__ void vision_rope_kernel(__nv_bfloat16* __restrict__ x, int N, int heads, int hd, int n_w, float theta) {
  const int half = hd / 2;
  const long long total = (long long)N * heads * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % half);
    const long long nh = i / half;
    const int n = (int)(nh / heads);
    const float pos = (k & 1) ? (float)(n % n_w) : (float)(n / n_w);
    const float inv = powf(theta, -2.0f * (float)(k >> 1) / (float)half);
    float s, c;
    sincosf(pos * inv, &s, &c);
    __nv_bfloat16* p = x + nh * hd;
    // the table is rounded to bf16 like the cached cos/sin of the tower
    c = __bfloat162float(__float2bfloat16(c)); s = __bfloat162float(__float2bfloat16(s));
    const float a = __bfloat162float(p[k]), b = __bfloat162float(p[k + half]);
    p[k] = __float2bfloat16(a * c - b * s);
    p[k + half] = __float2bfloat16(b * c + a * s);
  }
}

// x: [n_h, n_w, C] -> out [ceil(n_h/3) * ceil(n_w/3), C * 9], element c * 9 + kh * 3 + kw, zero padded
__global__ void vision_unfold3_kernel(const __nv_bfloat16* __restrict__ x, int n_h, int n_w, int C, __nv_bfloat16* __restrict__ out) {
  const int lw = (n_w + 2) / 3, lh = (n_h + 2) / 3;
  const long long total = (long long)lw * lh * C * 9;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int e = (int)(i % (C * 9));
    const long long cell = i / (C * 9);
    const int c = e / 9, kh = (e % 9) / 3, kw = e % 3;
    const int y = (int)(cell / lw) * 3 + kh, xx = (int)(cell % lw) * 3 + kw;
    out[i] = (y < n_h && xx < n_w) ? x[((size_t)y * n_w + xx) * C + c] : __float2bfloat16(0.f);
  }
}

}  // namespace sfb

extern "C" {

int sfb_vision_prepare(const void* img, int W, int H, int x0, int y0, int w, int h, int dw, int dh, int P, int grey, void* out, void* stream) {
  if (dw % P || dh % P) return 1;
  long long total = (long long)dw * dh * 3;
  int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  sfb::vision_prepare_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)img, W, H, x0, y0, w, h, dw, dh, P, grey, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}
int sfb_vision_rope(void* x, int N, int heads, int hd, int n_w, float theta, void* stream) {
  sfb::vision_rope_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, N, heads, hd, n_w, theta);
  return (int)cudaGetLastError();
}
int sfb_vision_unfold3(const void* x, int n_h, int n_w, int C, void* out, void* stream) {
  sfb::vision_unfold3_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, n_h, n_w, C, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

}  // extern "C"
