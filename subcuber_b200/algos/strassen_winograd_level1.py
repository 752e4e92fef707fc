"""One level of Strassen-Winograd written in the expression DSL.

The arithmetic contract of the whole path (reference: src/algos/strassen_winograd_level1.py:3-47):
quadrants are numbered row-major (0 top-left, 1 top-right, 2 bottom-left, 3 bottom-right);

    presums   s1 = a2 + a3    s2 = s1 - a0    a02 = a0 - a2    a1s2 = a1 - s2
              b10 = b1 - b0   b31 = b3 - b1   s3 = b31 + b0    s3b2 = s3 - b2
    products  m0 = a0 b0   m1 = a1 b2   m2 = s2 s3   m3 = a02 b31   m4 = s1 b10   m5 = a1s2 b3   m6 = a3 s3b2
    postsums  v1 = m0 + m2   v2 = v1 + m3   v3 = v1 + m4
              c0 = m0 + m1   c1 = v3 + m5   c2 = v2 - m6   c3 = v2 + m4
"""
from ..dsl import Combine4x4, Matrix


def strassen_winograd(m, n, k):
    """Build the expression DAG for an m x k by k x n product.  Returns (c, [m0, ..., m6])."""
    a = Matrix((m, k))
    b = Matrix((k, n))
    hm, hn, hk = m // 2, n // 2, k // 2

    a0, a1 = a[:hm, :hk], a[:hm, hk:]
    a2, a3 = a[hm:, :hk], a[hm:, hk:]
    b0, b1 = b[:hk, :hn], b[:hk, hn:]
    b2, b3 = b[hk:, :hn], b[hk:, hn:]

    s1 = a2 + a3
    s2 = s1 - a0
    a02 = a0 - a2
    a1s2 = a1 - s2
    b10 = b1 - b0
    b31 = b3 - b1
    s3 = b31 + b0
    s3b2 = s3 - b2

    m0 = a0 @ b0
    m1 = a1 @ b2
    m2 = s2 @ s3
    m3 = a02 @ b31
    m4 = s1 @ b10
    m5 = a1s2 @ b3
    m6 = a3 @ s3b2

    v1 = m0 + m2
    v2 = v1 + m3
    v3 = v1 + m4

    c0 = m0 + m1
    c1 = v3 + m5
    c2 = v2 - m6
    c3 = v2 + m4

    c = Combine4x4([c0, c1, c2, c3])
    c.var_names(locals())
    return c, [m0, m1, m2, m3, m4, m5, m6]
