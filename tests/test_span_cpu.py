"""The stage-unit spans of the integer-MMA matmul (csrc/gemm_i8.cu): CTA c of C takes units [SU*c/C, SU*(c+1)/C); the
kernel finds the CTAs that share a row group with `owner(x) = ceil((x + 1) * C / SU) - 1`.  Checked here against a
brute-force search over many (SU, C)."""
from __future__ import annotations


def span_begin(SU: int, c: int, C: int) -> int:
    return SU * c // C


def owner(SU: int, x: int, C: int) -> int:
    return ((x + 1) * C + SU - 1) // SU - 1


def test_owner_matches_a_search_over_the_spans():
    for SU in list(range(1, 70)) + [148, 149, 512, 1000, 3584, 28672]:
        for C in (1, 2, 3, 7, 64, 132, 148):
            if C > SU:
                continue
            spans = [(span_begin(SU, c, C), span_begin(SU, c + 1, C)) for c in range(C)]
            assert spans[0][0] == 0 and spans[-1][1] == SU and all(b > a for a, b in spans)
            step = max(1, SU // 500)
            for x in list(range(0, SU, step)) + [SU - 1]:
                want = next(c for c, (a, b) in enumerate(spans) if a <= x < b)
                assert owner(SU, x, C) == want, (SU, C, x)
