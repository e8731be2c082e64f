"""Summarises a tick-kernel trace (the file named by OMNI_TICK_TRACE) per phase shape.

    OMNI_TICK_TRACE=trace.txt python bench.py --steps 32 --warmup 8 --no-cpu-baseline --no-replay
    python -m pega_omni_b200.trace_summary trace.txt

The library writes one line per phase of the last traced tick: the phase's shape, its barrier-to-barrier duration,
and — median and latest over the CTAs, in ns after the previous barrier completed — when the first activation tile
was in shared memory (x), when the first accumulator was complete (acc), when the CTA's share of the phase was
done (work) and when it saw the grid barrier complete (bar). This script adds the lines up per shape.
"""
import collections
import sys

NAMES = {0: "gemm", 1: "embed_norm", 2: "reduce_norm", 3: "add_norm", 4: "rope_attn", 5: "sample", 6: "reduce_silu"}


def summarise(path, top=32):
    lines = open(path).read().strip().split("\n")
    rows = [list(map(int, line.split())) for line in lines[1:]]
    agg = collections.defaultdict(lambda: [0] * 10)
    for r in rows:
        _, kind, n, k, tiles, splits, _bn, nrows, tile_n = r[:9]
        a = agg[(NAMES.get(kind, str(kind)), n, k, tiles, splits, nrows, tile_n)]
        a[0] += 1
        for i in range(9):
            a[1 + i] += r[9 + i]
    total = sum(v[1] for v in agg.values())
    out = ["phases %d, %.1f us per tick" % (len(rows), total / 1000)]
    out.append("%-44s %4s %6s | %5s %5s | %5s %5s | %5s %5s | %5s %5s | %7s %5s" % (
        "(phase, N, K, tiles, splits, rows, tile_n)", "n", "dur", "x_md", "x_mx", "ac_md", "ac_mx", "wk_md", "wk_mx",
        "br_md", "br_mx", "tot_us", "%"))
    for key, v in sorted(agg.items(), key=lambda kv: -kv[1][1])[:top]:
        n = v[0]
        f = [x / n / 1000 for x in v[1:]]
        out.append("%-44s %4d %6.2f | %5.2f %5.2f | %5.2f %5.2f | %5.2f %5.2f | %5.2f %5.2f | %7.1f %5.1f" % (
            str(key), n, f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], f[8], v[1] / 1000, 100.0 * v[1] / total))
    return "\n".join(out)


if __name__ == "__main__":
    print(summarise(sys.argv[1] if len(sys.argv) > 1 else "trace.txt"))
