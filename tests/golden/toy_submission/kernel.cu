// Toy source of the packaging fixture: never compiled, only embedded.  Non-ASCII on purpose: "µs → ok".
__global__ void scale(const float* in, float* out, long n) {
  long i = blockIdx.x * 256L + threadIdx.x;
  if (i < n) out[i] = 2.0f * in[i];
}
void launch_scale(const float* in, float* out, long n, void* stream) {
  scale<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, n);
}
