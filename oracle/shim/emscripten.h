// Stand-in for <emscripten.h> so the reference header compiles natively.
// The reference calls emscripten_sleep(1) every 50 rows (src/lyapunov_fractal.hpp:92-94)
// to yield to the browser event loop; natively that is a no-op.
#pragma once
static inline void emscripten_sleep(unsigned) {}
