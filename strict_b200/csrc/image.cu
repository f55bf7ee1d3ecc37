// Image workloads of the reference's samples as real kernels: the 5x5 box blur over RGB bytes
// whose CPU form the reference specifies and tests
// (Strict.Compiler.Assembly.Tests/BlurPerformanceTests.cs:85-141: interior pixels sum 25
// neighbours and divide by 25, edge pixels sum the neighbours inside the image and divide by
// their count, integer division, per channel), and AdjustBrightness
// (ImageProcessing/AdjustBrightness.strict:16: every colour gets `brightness` added to Red,
// Green and Blue) over the flat fp32 array-of-structs layout of
// Strict.Expressions/ValueArrayInstance.cs:9-16,204-218 (element i, member m at
// offset + i*FlatWidth + m). The reference's own CUDA "blur" is a byte copy
// (Strict.Compiler.Cuda.Tests/BlurPerformanceTests.cs:111-117).
//
// Both are HBM streams (one byte read and one written per byte of image; one float read and
// written per colour member). The blur is also close to the integer-issue limit, so the fast
// kernel keeps two 16-bit sums per 32-bit register (25 x 255 fits 16 bits, so packed adds never
// carry between the lanes), is separable (horizontal 5-sums per row, a sliding window of five
// rows down a column strip), shares the sums of neighbouring taps between outputs, and divides by
// 25 on the floating-point pipe, which the integer-bound kernel leaves idle.
#include "common.cuh"

namespace {

constexpr int BLUR_THREADS = 128; // threads per block, one 16-byte chunk of a row each

// Bytes i and i+1 of a window of 32-bit words as two 16-bit lanes (i is a compile-time constant
// after unrolling). Inside one word the zero bytes come from a zero second operand of the byte
// permute; a pair that straddles two words takes a mask instead.
__device__ __forceinline__ uint32_t pair_at(const uint32_t* w, int i) {
  const int word = i >> 2, s = i & 3;
  if (s < 3) return __byte_perm(w[word], 0u, (uint32_t)(s | (4 << 4) | ((s + 1) << 8) | (4 << 12)));
  return __byte_perm(w[word], w[word + 1], 3u | (4u << 8)) & 0x00FF00FFu;
}

// sum / 25 for sum <= 6375, exactly, in one fused multiply-add on the floating-point pipe (the
// kernel is bound by the integer pipe). The sum enters a float through its mantissa:
// f = 2^23 + 22 * 2^16 + s (bit pattern BLUR_MAGIC | s). With m = 0.04 rounded up to the next float,
// m * (2^23 + 22 * 2^16) = 393216.0278..., so m * f - 393216 = s / 25 + d with 0.0278 <= d < 0.0279
// for every s <= 6375: always inside [s/25, s/25 + 1/25), hence its floor is the quotient. Adding
// 1.5 * 2^23 - 393216 (an integer, exact as a float) with round-toward-zero leaves that floor in
// the low mantissa bits. Checked against integer division for all 6376 sums (tests).
constexpr uint32_t BLUR_MAGIC = 0x4B160000u;
__device__ __forceinline__ uint32_t div25_bits(uint32_t magic_bits) {
  return __float_as_uint(__fmaf_rz(__uint_as_float(magic_bits), __uint_as_float(0x3D23D70Bu), 12189696.0f));
}

// Interior of the image: rows [2, H-2), bytes [x0, x1) of every such row with x0 >= 16,
// x1 <= stride - 16, both multiples of 16. A thread owns 16 consecutive bytes of a row strip and
// walks `rows_per_block` output rows down, keeping the horizontal sums of the last five input
// rows; the loads of the next input row are issued before the current one is worked on. 72
// registers: seven blocks of 128 threads per SM.
__global__ void __launch_bounds__(BLUR_THREADS, 7) blur5x5_rgb8_interior_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                                             int64_t stride, int height, int64_t x0, int64_t x1, int rows_per_block) {
  const int64_t x = x0 + ((int64_t)blockIdx.x * BLUR_THREADS + threadIdx.x) * 16;
  if (x >= x1) return;
  const int row_begin = 2 + blockIdx.y * rows_per_block;
  int row_end = row_begin + rows_per_block;
  if (row_end > height - 2) row_end = height - 2;
  // h[r % 5][p]: horizontal 5-sums of input row r for output byte pairs p (bytes 2p, 2p+1 of the 16)
  uint32_t h[5][8];
  uint32_t v[8];
#pragma unroll
  for (int p = 0; p < 8; p++) v[p] = 0;
  // bytes x-16 .. x+31 of a row as three aligned 16-byte loads (the neighbours' loads of the same lines hit in L1)
  struct Row { uint4 a, b, c; };
  auto load_row = [&](int r) {
    const uint4* p = (const uint4*)(src + (int64_t)r * stride + x);
    return Row{__ldg(p - 1), __ldg(p), __ldg(p + 1)};
  };
  auto hsum_row = [&](const Row& in, uint32_t* out) {
    const uint32_t w[12] = {in.a.x, in.a.y, in.a.z, in.a.w, in.b.x, in.b.y, in.b.z, in.b.w, in.c.x, in.c.y, in.c.z, in.c.w};
    // Byte 0 of the window is x-16, so output byte j is window byte 16+j and its five taps are
    // window bytes 10+j, 13+j, 16+j, 19+j, 22+j; output pair q covers j = 2q, 2q+1. The sum of
    // two neighbouring taps, t(i) = pair(i) + pair(i+3), serves two outputs: out(q) = t(10+2q) + t(16+2q) + pair(22+2q),
    // and t(16+2q) is t(10+2(q+3)).
    uint32_t t[11];
#pragma unroll
    for (int i = 0; i < 11; i++) t[i] = pair_at(w, 10 + 2 * i) + pair_at(w, 13 + 2 * i);
#pragma unroll
    for (int q = 0; q < 8; q++) out[q] = t[q] + t[q + 3] + pair_at(w, 22 + 2 * q);
  };
  // prime the window with input rows row_begin-2 .. row_begin+1
  {
    Row r0 = load_row(row_begin - 2), r1 = load_row(row_begin - 1), r2 = load_row(row_begin), r3 = load_row(row_begin + 1);
    hsum_row(r0, h[0]); hsum_row(r1, h[1]); hsum_row(r2, h[2]); hsum_row(r3, h[3]);
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int p = 0; p < 8; p++) v[p] += h[i][p];
  }
  Row next = load_row(row_begin + 2);  // row_begin + 2 <= height - 1
  // five output rows per turn, so that every index into the ring of row sums is a constant
  for (int base = row_begin; base < row_end; base += 5) {
#pragma unroll
    for (int i = 0; i < 5; i++) {
      const int r = base + i;
      if (r < row_end) {
        const int slot = (i + 4) % 5;  // holds input row r+2 from now on; it held row r-3, already taken out of v
        const Row cur = next;
        if (r + 1 < row_end) next = load_row(r + 3);  // in flight while row r+2 is summed and row r is written
        hsum_row(cur, h[slot]);
        uint32_t q[4];
#pragma unroll
        for (int p = 0; p < 8; p += 2) {
          v[p] += h[slot][p];
          v[p + 1] += h[slot][p + 1];
          // the four sums of an output word as floats 2^23 + s: low lanes by mask, high lanes by byte permute
          const uint32_t b0 = div25_bits((v[p] & 0xFFFFu) | BLUR_MAGIC), b1 = div25_bits(__byte_perm(v[p], BLUR_MAGIC, 0x7632));
          const uint32_t b2 = div25_bits((v[p + 1] & 0xFFFFu) | BLUR_MAGIC), b3 = div25_bits(__byte_perm(v[p + 1], BLUR_MAGIC, 0x7632));
          q[p >> 1] = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
        }
        __stcs((uint4*)(dst + (int64_t)r * stride + x), make_uint4(q[0], q[1], q[2], q[3]));  // written once, not read again by this kernel
#pragma unroll
        for (int p = 0; p < 8; p++) v[p] -= h[i][p];  // input row r-2 leaves the window
      }
    }
  }
}

// Any byte of the image, exactly as the reference's edge path computes it (which equals its
// interior path where all 25 neighbours exist). One thread per byte of the listed region:
// region 0 = rows [0,2) and [H-2,H) in full; region 1 = bytes [0,xa) and [xb,stride) of rows [2,H-2).
__global__ void blur5x5_rgb8_generic_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int width, int height,
                                            int64_t xa, int64_t xb, int64_t total) {
  const int64_t stride = (int64_t)width * 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    // decode i into (row, byte in row)
    int row;
    int64_t xbyte;
    const int border_rows = height < 4 ? height : 4;
    const int64_t top = (int64_t)border_rows * stride;
    if (i < top) {
      int r = (int)(i / stride);
      xbyte = i - (int64_t)r * stride;
      const int upper = height < 4 ? height : 2;
      row = r < upper ? r : height - border_rows + r;  // rows 0,1 then H-2,H-1
    } else {
      const int64_t per_row = xa + (stride - xb), j = i - top;
      row = 2 + (int)(j / per_row);
      const int64_t k = j - (int64_t)(row - 2) * per_row;
      xbyte = k < xa ? k : xb + (k - xa);
    }
    const int column = (int)(xbyte / 3), channel = (int)(xbyte - (int64_t)column * 3);
    int sum = 0, count = 0;
    for (int ky = -2; ky <= 2; ky++)
      for (int kx = -2; kx <= 2; kx++) {
        const int nx = column + kx, ny = row + ky;
        if ((unsigned)nx >= (unsigned)width || (unsigned)ny >= (unsigned)height) continue;
        sum += src[(int64_t)ny * stride + (int64_t)nx * 3 + channel];
        count++;
      }
    dst[(int64_t)row * stride + xbyte] = (uint8_t)(sum / count);
  }
}

// flat[offset + i*fw + m] += brightness for m < channels, i < count; the sum is taken in double
// and rounded to float once, as the reference's VM does (doubles in registers, a float[] store).
__global__ void adjust_brightness_kernel(float* __restrict__ flat, int64_t offset, int64_t count, int fw, int channels, double brightness, int clamp01) {
  const int64_t total = count * fw, step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += step) {
    const int m = (int)(j % fw);
    if (m >= channels) continue;
    double s = (double)flat[offset + j] + brightness;
    if (clamp01) s = s < 0.0 ? 0.0 : (s > 1.0 ? 1.0 : s);
    flat[offset + j] = (float)s;
  }
}
// FlatWidth 4 (Color = Red, Green, Blue, Alpha) with a 16-byte aligned first element: one 128-bit load and store per colour.
__global__ void adjust_brightness_rgba_kernel(float4* __restrict__ colors, int64_t count, int channels, double brightness, int clamp01) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
    float4 c = colors[i];
    float* f = &c.x;
#pragma unroll
    for (int m = 0; m < 4; m++)
      if (m < channels) {
        double s = (double)f[m] + brightness;
        if (clamp01) s = s < 0.0 ? 0.0 : (s > 1.0 ? 1.0 : s);
        f[m] = (float)s;
      }
    colors[i] = c;
  }
}

}  // namespace

int k_blur5x5_rgb8(strictb200_ctx* ctx, const uint8_t* src, uint8_t* dst, int width, int height) {
  const int64_t stride = (int64_t)width * 3;
  // bytes [xa, xb) of rows [2, H-2) go to the strip kernel: whole 16-byte chunks inside [6, stride-6), readable with aligned 128-bit loads
  int64_t xa = 16, xb = (stride - 6) / 16 * 16;
  const bool fast = height > 4 && stride % 16 == 0 && xb > xa && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0;
  if (!fast) xa = xb = stride;  // everything through the generic kernel (xa bytes on the left, none on the right)
  if (fast) {
    const int64_t chunks = (xb - xa) / 16, strips = (chunks + BLUR_THREADS - 1) / BLUR_THREADS;
    // Rows per block. A block reads four rows of halo again and sums them again, so taller blocks
    // do less work in total; measured on 8192 x 8192 they are slower all the same (111 us at 8 rows,
    // 113 at 16, 119 at 32, 134 at 64, 138 at 128): with short blocks the blocks that run at one
    // time cover a narrow band of the image that moves down it, the halo rows are found in L2, and
    // small images still give every SM several blocks. The option blur_rows overrides the choice.
    const int rows = ctx->opt.blur_rows > 0 ? ctx->opt.blur_rows : 8;
    dim3 grid((unsigned)strips, (unsigned)((height - 4 + rows - 1) / rows));
    if (grid.y > 65535) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "blur: too many blocks of rows for one launch (raise the option blur_rows)");
    blur5x5_rgb8_interior_kernel<<<grid, BLUR_THREADS, 0, ctx->stream>>>(src, dst, stride, height, xa, xb, rows);
    SB_LAUNCHED(ctx);
  }
  const int border_rows = height < 4 ? height : 4;
  const int64_t total = (int64_t)border_rows * stride + (height > 4 ? (int64_t)(height - 4) * (xa + stride - xb) : 0);
  if (total > 0) {
    int64_t blocks = (total + 255) / 256, cap = (int64_t)ctx->sm_count * 16;
    blur5x5_rgb8_generic_kernel<<<(unsigned)(blocks > cap ? cap : blocks), 256, 0, ctx->stream>>>(src, dst, width, height, xa, xb, total);
    SB_LAUNCHED(ctx);
  }
  return STRICTB200_OK;
}

int k_adjust_brightness(strictb200_ctx* ctx, float* flat, int64_t offset, int64_t count, int fw, int channels, double brightness, int clamp01) {
  if (fw == 4 && (((uintptr_t)(flat + offset)) & 15) == 0) {
    int64_t blocks = (count + 255) / 256, cap = (int64_t)ctx->sm_count * 16;
    adjust_brightness_rgba_kernel<<<(unsigned)(blocks > cap ? cap : blocks), 256, 0, ctx->stream>>>((float4*)(flat + offset), count, channels, brightness, clamp01);
  } else {
    int64_t blocks = (count * fw + 255) / 256, cap = (int64_t)ctx->sm_count * 16;
    adjust_brightness_kernel<<<(unsigned)(blocks > cap ? cap : blocks), 256, 0, ctx->stream>>>(flat, offset, count, fw, channels, brightness, clamp01);
  }
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}

extern "C" {

int strictb200_blur5x5_rgb8(strictb200_ctx* ctx, const uint8_t* d_src, uint8_t* d_dst, int width, int height) {
  SB_ENTER(ctx);
  SB_REQUIRE(width >= 0 && height >= 0, "negative size");
  if (!width || !height) return STRICTB200_OK;
  SB_REQUIRE(d_src && d_dst && d_src != d_dst, "source and destination must be two different buffers");
  return k_blur5x5_rgb8(ctx, d_src, d_dst, width, height);
}

int strictb200_adjust_brightness(strictb200_ctx* ctx, float* d_flat, int64_t offset, int64_t count, int flat_width, int channels,
                                 double brightness, int clamp01) {
  SB_ENTER(ctx);
  SB_REQUIRE(offset >= 0 && count >= 0 && flat_width >= 1 && channels >= 0 && channels <= flat_width, "bad layout");
  if (!count || !channels) return STRICTB200_OK;
  SB_REQUIRE(d_flat, "null pointer");
  return k_adjust_brightness(ctx, d_flat, offset, count, flat_width, channels, brightness, clamp01);
}

}  // extern "C"
