// Which two columns of a head make rotary pair i, for the two usual layouts, and the rotation.
#pragma once

// halves: pair i = (i, i + rot_half), the split-halves layout; interleaved: pair i = (2i, 2i + 1).
__device__ __forceinline__ void rotary_pair(int i, int rot_half, int interleaved, int& a, int& b) {
    a = interleaved ? 2 * i : i;
    b = interleaved ? 2 * i + 1 : i + rot_half;
}

// (u, v) turned by the angle whose cosine and sine are c and s.
__device__ __forceinline__ void rotate(float u, float v, float c, float s, float& ru, float& rv) {
    ru = u * c - v * s;
    rv = v * c + u * s;
}
