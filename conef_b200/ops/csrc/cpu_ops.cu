// Host (CPU) implementations of the sketch primitives and Gram-Schmidt.
// They serve the gloo / CPU execution path and double as a second oracle for
// the device kernels (same hash arithmetic, plain loops, fp32).
// Spec: communication/compressors/CountSketch.py:7-98 and
// communication/powerSGD_hook.py:12-43 of the reference.
#include <math.h>
#include <string.h>
#include <vector>
#include "common.cuh"

extern "C" void conef_cpu_hash_table(int32_t* table, int32_t* counts, int D, int W, int a, int b, int sa, int sb,
                                     int layout) {
  if (counts) memset(counts, 0, sizeof(int32_t) * (size_t)W);
  for (int j = 0; j < D; ++j) {
    const int h = conef_cell(j, W, a, b, layout);
    const int sign_bit = conef_hash(j, W, a + sa, b + sb) & 1;
    table[j] = (int32_t)((uint32_t)h | ((uint32_t)sign_bit << 31));
    if (counts) counts[h] += 1;
  }
}

extern "C" void conef_cpu_sketch_query(float* mat, const float* cs, const int32_t* table, int N, int D, int W,
                                       float alpha) {
  for (int i = 0; i < N; ++i) {
    float* row = mat + (size_t)i * D;
    const float* srow = cs + (size_t)i * W;
    for (int j = 0; j < D; ++j) {
      const int e = table[j];
      const float s = e < 0 ? 1.f : -1.f;
      row[j] += alpha * s * srow[e & 0x7fffffff];
    }
  }
}

extern "C" void conef_cpu_sketch_update(const float* vec, float* cs, const int32_t* table, const int32_t* counts,
                                        int N, int D, int W, float beta) {
  std::vector<float> acc((size_t)W);
  const float omb = 1.f - beta;
  for (int i = 0; i < N; ++i) {
    std::fill(acc.begin(), acc.end(), 0.f);
    const float* row = vec + (size_t)i * D;
    for (int j = 0; j < D; ++j) {
      const int e = table[j];
      acc[e & 0x7fffffff] += (e < 0 ? 1.f : -1.f) * row[j];
    }
    float* srow = cs + (size_t)i * W;
    for (int h = 0; h < W; ++h) srow[h] = srow[h] * (1.f - omb * (float)counts[h]) + acc[h];
  }
}

extern "C" void conef_cpu_gram_schmidt(float* mat, int rows, int cols, float eps) {
  for (int c = 0; c < cols; ++c) {
    double nn = 0.0;
    for (int i = 0; i < rows; ++i) nn += (double)mat[(size_t)i * cols + c] * mat[(size_t)i * cols + c];
    const float inv = 1.f / ((float)sqrt(nn) + eps);
    for (int i = 0; i < rows; ++i) mat[(size_t)i * cols + c] *= inv;
    for (int d = c + 1; d < cols; ++d) {
      double dot = 0.0;
      for (int i = 0; i < rows; ++i) dot += (double)mat[(size_t)i * cols + c] * mat[(size_t)i * cols + d];
      const float f = (float)dot;
      for (int i = 0; i < rows; ++i) mat[(size_t)i * cols + d] -= f * mat[(size_t)i * cols + c];
    }
  }
}
