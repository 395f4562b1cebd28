// Gated activations of a feed-forward, y = act(gate, up), shared by the row-wise kernel and the
// epilogues of the experts' products.
//   GLU_SILU      silu(g) * u
//   GLU_CLAMPED   g = min(g, limit), u = clamp(u, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1)
#pragma once

enum { GLU_SILU = 0, GLU_CLAMPED = 1 };

// What an epilogue needs to know of the activation; kind GLU_SILU ignores the rest.
struct GluArgs { int kind; float limit, alpha; };

__device__ __forceinline__ float glu_activation(int kind, float g, float u, float limit, float alpha) {
    if (kind == GLU_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    }
    return g / (1.0f + expf(-g)) * u;
}
