"""Known answers of the checker's SwiGLU (binary64): silu(g) * u with silu(g) = g / (1 + exp(-g))."""
import math

import numpy as np


def test_swiglu_known_answers(orc):
    gu = np.array([[0.0, 1.0, -1.0, 50.0, -50.0, 800.0, -800.0,      # gate
                    5.0, 2.0, 2.0, 1.0, 1.0, 3.0, 3.0]])            # up
    h = orc.swiglu_f64(gu)[0]
    e = math.e
    want = [0.0, 2.0 / (1.0 + 1.0 / e), -2.0 / (1.0 + e), 50.0 / (1.0 + math.exp(-50.0)), -50.0 / (1.0 + math.exp(50.0)), 2400.0, -0.0]
    assert np.allclose(h, want, rtol=1e-15, atol=0.0)
    assert h[6] == 0.0 and np.isfinite(h).all()                      # exp overflows to +inf: the quotient is a signed zero
    # the minimum of silu, about -0.27846 at g = -1.27846
    g = np.linspace(-3.0, 0.0, 300001)
    s = orc.swiglu_f64(np.stack([g, np.ones_like(g)], axis=0).T.reshape(-1, 2))[:, 0]
    assert abs(s.min() + 0.2784645427610738) < 1e-9 and abs(g[s.argmin()] + 1.2784645427610738) < 1e-4
