"""One level of Strassen's original algorithm written in the expression DSL.

The second <2,2,2;7> algorithm of this package (the reference lists "other Strassen-like algorithms through the DSL" as
future work, README.md:179, and keeps its C++ side stubbed, include/cutlass/gemm/kernel/strassen_gemm.h:1360-1398).
Quadrants are numbered row-major as in strassen_winograd_level1.py.

    products  m1 = (a0 + a3)(b0 + b3)   m2 = (a2 + a3) b0   m3 = a0 (b1 - b3)   m4 = a3 (b2 - b0)
              m5 = (a0 + a1) b3         m6 = (a2 - a0)(b0 + b1)                 m7 = (a1 - a3)(b2 + b3)
    postsums  c0 = m1 + m4 - m5 + m7    c1 = m3 + m5    c2 = m2 + m4    c3 = m1 - m2 + m3 + m6

18 additions against Strassen-Winograd's 15, but no operand sums more than two quadrants, so every presum can be
formed on the fly from two shared-memory tiles.
"""
from ..dsl import Combine4x4, Matrix


def strassen(m, n, k):
    """Build the expression DAG for an m x k by k x n product.  Returns (c, [m1, ..., m7])."""
    a = Matrix((m, k))
    b = Matrix((k, n))
    hm, hn, hk = m // 2, n // 2, k // 2

    a0, a1 = a[:hm, :hk], a[:hm, hk:]
    a2, a3 = a[hm:, :hk], a[hm:, hk:]
    b0, b1 = b[:hk, :hn], b[:hk, hn:]
    b2, b3 = b[hk:, :hn], b[hk:, hn:]

    a03 = a0 + a3
    a23 = a2 + a3
    a01 = a0 + a1
    a20 = a2 - a0
    a13 = a1 - a3
    b03 = b0 + b3
    b13 = b1 - b3
    b20 = b2 - b0
    b01 = b0 + b1
    b23 = b2 + b3

    m1 = a03 @ b03
    m2 = a23 @ b0
    m3 = a0 @ b13
    m4 = a3 @ b20
    m5 = a01 @ b3
    m6 = a20 @ b01
    m7 = a13 @ b23

    c0 = ((m1 + m4) - m5) + m7
    c1 = m3 + m5
    c2 = m2 + m4
    c3 = ((m1 - m2) + m3) + m6

    c = Combine4x4([c0, c1, c2, c3])
    c.var_names(locals())
    return c, [m1, m2, m3, m4, m5, m6, m7]
