// Toy header of the packaging fixture: never compiled, only embedded.
#pragma once
void launch_scale(const float* in, float* out, long n, void* stream);
