"""Turn the JSON lines of ``bench/sparse_microbench.py`` (multi-GPU mode) into a markdown table with roofline bounds.

    python bench/sparse_table.py out1.jsonl [out2.jsonl ...] [--hbm_gbs 6542] [--link_gbs 770]

Bounds per call and rank: the HBM term is "read the bucket once and write the result once" at the measured copy rate;
the NVLink term is the larger of the bytes this rank sends and the bytes it receives (records to the owners, then the
gathered runs from every other owner) at the measured peer-copy rate per direction.  ``achieved`` is the slower bound
divided by the measured time.
"""
import argparse
import json


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--hbm_gbs", type=float, default=6542.1)
    ap.add_argument("--link_gbs", type=float, default=770.0)
    args = ap.parse_args()
    rows = []
    for f in args.files:
        for line in open(f):
            line = line.strip()
            if line.startswith("{"):
                r = json.loads(line)
                if r.get("mode") == "nvlink":
                    rows.append(r)
    print("| GPUs | dtype | elements | density | indices | overlap | transport | sparse, us | dense NCCL, us | speed-up | "
          "reference m3 / m2 / m1, us | union density | format | NVLink bytes / rank | NVLink bound, us | HBM bound, us | achieved |")
    print("|" + "---|" * 17)
    for r in rows:
        es = 2 if r["dtype"] == "bf16" else 4
        n = 1 << r["log2n"]
        P = r["P"]
        rec_out = r.get("push_bytes_per_rank", 0.0)
        gath = r.get("gather_bytes_pushed", 0.0)                 # (P - 1) x this owner's run: what a rank receives in total
        link_bytes = rec_out + gath
        t_link = link_bytes / (args.link_gbs * 1e3)              # us
        t_hbm = 2.0 * n * es / (args.hbm_gbs * 1e3)
        bound = max(t_link, t_hbm)
        us = r["sparse_ms"] * 1e3
        ref = " / ".join(f"{r[k] * 1e3:.0f}" if isinstance(r.get(k), float) else "-" for k in
                         ("reference_m3_ms", "reference_m2_ms", "reference_m1_ms"))
        print(f"| {P} | {r['dtype']} | 2^{r['log2n']} | {r['density'] * 100:g} % | {r['dist']} | {r['overlap'] * 100:g} % | "
              f"{r.get('transport', 'p2p')} | {us:.0f} | {r['dense_nccl_ms'] * 1e3:.0f} | {r['speedup']:.2f}x | {ref} | "
              f"{r.get('union_density', float('nan')) * 100:.1f} % | {r.get('format', '-')} | {link_bytes / 1e6:.1f} MB | "
              f"{t_link:.0f} | {t_hbm:.0f} | {bound / us * 100:.0f} % |")


if __name__ == "__main__":
    main()
