"""Analysis of benchmark CSVs (the schema ``bench/driver.py`` and the reference
write): median per cell, winner per ``(nprocs, send_count)``, speed-up over the
library collective.  Headless: matplotlib's Agg backend, figures are saved.

    python -m configurable_hierarchical_allreduce_algorithms_b200.bench.plots median_best  results.csv [--outdir DIR]
    python -m ...bench.plots per_algo     results.csv [--outdir DIR]      # one PNG per nprocs, time vs size
    python -m ...bench.plots radix        results.csv [--outdir DIR]      # median time vs k per send_count
    python -m ...bench.plots winners      results.csv [--outdir DIR]      # log-log lines of the winning k only

Counterparts in the reference: testing/plots/all_reduce/median_best_plotter.py:1-140 (winner grid,
refusal of rows with is_correct != 1 at :15-20, baseline / best-of-mine speed-up at :53-56),
testing/plots/reduce_scatter/make_median_algo_plot.py:47-90, testing/plots/all_gather/
fixed_sendcount_procs_plotter.py:41-104, testing/plots/all_gather/median_plotter.py:62-96,
and the mean / minimum variants (avg_best_plotter.py, minimum_best_plotter.py) via ``--stat``.
"""
from __future__ import annotations

import argparse
import os

import numpy as np
import pandas as pd

try:  # matplotlib is optional: without it the winner grid is written as a markdown table
    import matplotlib

    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
except ImportError:  # pragma: no cover - depends on the image
    plt = None


def _md_table(path: str, header: list[str], rows: list[list]) -> str:
    """Without matplotlib every analysis is written as a markdown table instead of a figure."""
    with open(path, "w") as f:
        f.write("| " + " | ".join(header) + " |\n|" + "---|" * len(header) + "\n")
        for r in rows:
            f.write("| " + " | ".join(f"{v:.3e}" if isinstance(v, float) else str(v) for v in r) + " |\n")
    return path


VENDOR_NAMES = {"MPICH_allreduce", "allgather_standard", "reduce_scatter_standard"}
# The tuner's CSV (bench/tune.py --csv) names its rows <collective>_<kernel or schedule>; the library rows there are
# NCCL's default choice and NCCL pinned to ring / tree.  FILTER narrows such a file (all collectives, two dtypes)
# to one collective and dtype before any statistic is taken.
TUNER_VENDOR_SUFFIXES = ("_nccl", "_nccl_ring", "_nccl_tree")
FILTER = {"coll": "", "dtype": ""}


def is_vendor(name: str) -> bool:
    return name in VENDOR_NAMES or name.endswith(TUNER_VENDOR_SUFFIXES)


def is_vendor_default(name: str) -> bool:
    """The library's own choice (what the speed-up is taken against), not one of its pinned variants."""
    return name in VENDOR_NAMES or name.endswith("_nccl")


def load(path: str) -> pd.DataFrame:
    df = pd.read_csv(path)
    if FILTER["coll"]:
        df = df[df["algorithm_name"].str.startswith(FILTER["coll"] + "_")]
    if FILTER["dtype"] and "dtype" in df.columns:
        df = df[df["dtype"] == FILTER["dtype"]]
    df = df.reset_index(drop=True)
    bad = df[df["is_correct"] != 1]
    if len(bad):
        raise SystemExit(f"{len(bad)} rows of {path} have is_correct != 1; refusing to plot:\n{bad.head()}")
    if "b" not in df.columns:
        df["b"] = 0
    if "nctas" in df.columns:     # the tuner's file: a candidate is a shape (k, b) at a CTA count
        df["label"] = np.where(df["k"] > 0, df["algorithm_name"] + " (k=" + df["k"].astype(str) + ", b=" + df["b"].astype(str) +
                               ", ctas=" + df["nctas"].astype(str) + ")", df["algorithm_name"])
    else:
        df["label"] = np.where(df["k"] > 0, df["algorithm_name"] + " (k=" + df["k"].astype(str) + ")", df["algorithm_name"])
    return df


def cell_stat(df: pd.DataFrame, stat: str = "median") -> pd.DataFrame:
    g = df.groupby(["nprocs", "send_count", "label", "algorithm_name"])["time"]
    return getattr(g, stat)().reset_index()


def winners_table(df: pd.DataFrame, stat: str = "median") -> pd.DataFrame:
    """One row per (nprocs, send_count): best own label, its time, vendor time, speed-up."""
    m = cell_stat(df, stat)
    rows = []
    for (p, n), g in m.groupby(["nprocs", "send_count"]):
        mine = g[~g["algorithm_name"].map(is_vendor)]
        vend = g[g["algorithm_name"].map(is_vendor_default)]
        if not len(mine):
            continue
        best = mine.loc[mine["time"].idxmin()]
        vt = float(vend["time"].min()) if len(vend) else float("nan")
        rows.append({"nprocs": p, "send_count": n, "winner": best["label"], "time": float(best["time"]),
                     "vendor_time": vt, "speedup": vt / float(best["time"]) if vt == vt else float("nan")})
    return pd.DataFrame(rows)


def median_best(path: str, outdir: str = ".", stat: str = "median") -> str:
    df = load(path)
    w = winners_table(df, stat)
    labels = sorted(w["winner"].unique())
    ps, ns = sorted(w["nprocs"].unique()), sorted(w["send_count"].unique())
    if plt is None:
        out = os.path.join(outdir, f"{stat}_best_" + os.path.splitext(os.path.basename(path))[0] + ".md")
        with open(out, "w") as f:
            f.write("| nprocs | send_count | winner | time (s) | library (s) | speed-up |\n|---|---|---|---|---|---|\n")
            for _, r in w.sort_values(["nprocs", "send_count"]).iterrows():
                f.write(f"| {r['nprocs']} | {r['send_count']} | {r['winner']} | {r['time']:.3e} | "
                        f"{r['vendor_time']:.3e} | {r['speedup']:.2f}x |\n")
        return out
    grid = np.full((len(ps), len(ns)), np.nan)
    for _, r in w.iterrows():
        grid[ps.index(r["nprocs"]), ns.index(r["send_count"])] = labels.index(r["winner"])
    fig, ax = plt.subplots(figsize=(max(6, 1.2 * len(ns)), max(3, 0.8 * len(ps) + 2)))
    cmap = plt.get_cmap("tab20", max(1, len(labels)))
    ax.pcolormesh(grid, cmap=cmap, vmin=-0.5, vmax=len(labels) - 0.5, edgecolors="k", linewidth=0.5)
    for _, r in w.iterrows():
        if r["speedup"] == r["speedup"]:
            ax.text(ns.index(r["send_count"]) + 0.5, ps.index(r["nprocs"]) + 0.5, f"{r['speedup']:.2f}x",
                    ha="center", va="center", fontsize=8)
    ax.set_xticks(np.arange(len(ns)) + 0.5, [str(n) for n in ns], rotation=45)
    ax.set_yticks(np.arange(len(ps)) + 0.5, [str(p) for p in ps])
    ax.set_xlabel("send_count (elements per rank)")
    ax.set_ylabel("nprocs")
    ax.set_title(f"{stat} winner per cell; number = library time / winner time")
    ax.legend(handles=[plt.Rectangle((0, 0), 1, 1, color=cmap(i)) for i in range(len(labels))], labels=labels,
              bbox_to_anchor=(1.01, 1), loc="upper left", fontsize=7)
    out = os.path.join(outdir, f"{stat}_best_" + os.path.splitext(os.path.basename(path))[0] + ".png")
    fig.savefig(out, dpi=120, bbox_inches="tight")
    plt.close(fig)
    return out


def per_algo(path: str, outdir: str = ".", stat: str = "median") -> list[str]:
    m = cell_stat(load(path), stat)
    outs = []
    for p, g in m.groupby("nprocs"):
        if plt is None:
            best = g.groupby(["send_count", "algorithm_name"])["time"].min().unstack("algorithm_name")
            rows = [[int(n)] + [float(v) if v == v else "" for v in best.loc[n].values] for n in best.index]
            outs.append(_md_table(os.path.join(outdir, f"{stat}_per_algo_np{p}.md"), ["send_count"] + list(best.columns), rows))
            continue
        fig, ax = plt.subplots(figsize=(7, 4.5))
        for name, h in g.groupby("algorithm_name"):
            best = h.groupby("send_count")["time"].min()
            ax.plot(best.index, best.values, marker="o", ms=3, label=name, ls="--" if is_vendor(name) else "-")
        ax.set_xscale("log", base=2)
        ax.set_yscale("log")
        ax.set_xlabel("send_count / rank")
        ax.set_ylabel(f"{stat} time (s)")
        ax.set_title(f"nprocs = {p}")
        ax.legend(fontsize=6)
        out = os.path.join(outdir, f"{stat}_per_algo_np{p}.png")
        fig.savefig(out, dpi=120, bbox_inches="tight")
        plt.close(fig)
        outs.append(out)
    return outs


def radix(path: str, outdir: str = ".", stat: str = "median") -> str:
    """Median time against k for every send_count; best / second / worst k marked, library as a dashed line."""
    df = load(path)
    ns = sorted(df["send_count"].unique())
    if plt is None:
        rows = []
        for n in ns:
            g = df[(df["send_count"] == n) & (df["k"] > 0)]
            order = getattr(g.groupby("k")["time"], stat)().sort_values()
            v = df[(df["send_count"] == n) & df["algorithm_name"].map(is_vendor_default)]["time"]
            rows.append([int(n), int(order.index[0]) if len(order) else "", float(order.iloc[0]) if len(order) else "",
                         int(order.index[1]) if len(order) > 1 else "", int(order.index[-1]) if len(order) > 1 else "",
                         float(getattr(v, stat)()) if len(v) else ""])
        return _md_table(os.path.join(outdir, "radix_" + os.path.splitext(os.path.basename(path))[0] + ".md"),
                         ["send_count", "best k", "its time (s)", "second k", "worst k", "library (s)"], rows)
    fig, axes = plt.subplots(1, len(ns), figsize=(3.2 * len(ns), 3), squeeze=False)
    for ax, n in zip(axes[0], ns):
        g = df[(df["send_count"] == n) & (df["k"] > 0)]
        med = getattr(g.groupby("k")["time"], stat)()
        ax.plot(med.index, med.values, marker="o", ms=3)
        if len(med):
            order = med.sort_values()
            ax.scatter([order.index[0]], [order.iloc[0]], c="g", zorder=3, label="best")
            if len(order) > 1:
                ax.scatter([order.index[1]], [order.iloc[1]], c="orange", zorder=3, label="second")
                ax.scatter([order.index[-1]], [order.iloc[-1]], c="r", zorder=3, label="worst")
        v = df[(df["send_count"] == n) & df["algorithm_name"].map(is_vendor_default)]["time"]
        if len(v):
            ax.axhline(getattr(v, stat)(), ls="--", c="k", lw=0.8)
        ax.set_title(f"send_count {n}", fontsize=8)
        ax.set_xlabel("k")
    axes[0][0].set_ylabel(f"{stat} time (s)")
    out = os.path.join(outdir, "radix_" + os.path.splitext(os.path.basename(path))[0] + ".png")
    fig.savefig(out, dpi=120, bbox_inches="tight")
    plt.close(fig)
    return out


def winners(path: str, outdir: str = ".", stat: str = "median") -> str:
    df = load(path)
    w = winners_table(df, stat)
    if plt is None:
        rows = [[int(r["nprocs"]), int(r["send_count"]), r["winner"], float(r["time"]), float(r["vendor_time"])]
                for _, r in w.sort_values(["nprocs", "send_count"]).iterrows()]
        return _md_table(os.path.join(outdir, "winners_" + os.path.splitext(os.path.basename(path))[0] + ".md"),
                         ["nprocs", "send_count", "winner", "time (s)", "library (s)"], rows)
    fig, ax = plt.subplots(figsize=(7, 4.5))
    for p, g in w.groupby("nprocs"):
        g = g.sort_values("send_count")
        ax.plot(g["send_count"], g["time"], marker="o", ms=3, label=f"np={p} best")
        ax.plot(g["send_count"], g["vendor_time"], ls="--", lw=0.8, label=f"np={p} library")
    ax.set_xscale("log", base=2)
    ax.set_yscale("log")
    ax.set_xlabel("send_count / rank")
    ax.set_ylabel(f"{stat} time (s)")
    ax.legend(fontsize=6)
    out = os.path.join(outdir, "winners_" + os.path.splitext(os.path.basename(path))[0] + ".png")
    fig.savefig(out, dpi=120, bbox_inches="tight")
    plt.close(fig)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["median_best", "per_algo", "radix", "winners"])
    ap.add_argument("csv")
    ap.add_argument("--outdir", default=".")
    ap.add_argument("--stat", default="median", choices=["median", "mean", "min"])
    ap.add_argument("--coll", default="", help="keep only rows of this collective (for the tuner's CSV, which holds all three)")
    ap.add_argument("--dtype", default="", help="keep only rows of this dtype (column dtype, if the file has one)")
    a = ap.parse_args(argv)
    FILTER.update(coll=a.coll, dtype=a.dtype)
    os.makedirs(a.outdir, exist_ok=True)
    print({"median_best": median_best, "per_algo": per_algo, "radix": radix, "winners": winners}[a.what](a.csv, a.outdir, a.stat))


if __name__ == "__main__":
    main()
