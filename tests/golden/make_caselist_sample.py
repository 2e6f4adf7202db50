"""Distils the reference's case corpus (caselist/decode/*.list, caselist/prefill/*.list in the reference tree:
56,659 GDN/KDA records plus Mamba2 ones this library does not serve) into two small committed files:

* ``corpus_census.json`` -- per shape group (operator, phase, key heads, value heads, dtype, query length, gate
  lower bound): how many records, how many distinct batch sizes, the smallest / median / largest token count.
  ``tests/test_caselist.py`` recomputes it whenever the reference tree is present, which proves that the parser
  reads every record of the corpus.
* ``corpus_sample.list`` -- a few records per group, verbatim in the corpus grammar: for decode groups the largest
  batch and one more picked by a hash of the group; for prefill groups the shortest batch, the one with the most
  sequences, one picked by hash, and for every fourth group the longest. The GPU test replays each of them and
  checks a head subset against the CPU oracle.

Usage:  python tests/golden/make_caselist_sample.py /path/to/reference/caselist
"""
import hashlib
import json
import sys
from collections import defaultdict
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from pla_b200 import caselist as cl   # noqa: E402

SERVED = ("gdn_attn", "kda_attn")


def group_key(c):
    return "|".join(str(x) for x in (c["op"], c["phase"], c.get("num_heads_qk"), c.get("num_heads_v"), c["dtype"],
                                     c.get("seqlen_q"), c.get("gate_lower_bound")))


def tokens_of(c):
    offs = cl.offsets_of(c) if c["phase"] == "P" else None
    return offs[-1] if offs else int(c["batch_size"]) * int(c.get("seqlen_q", 1))


def walk(root):
    """Every record of every list below ``root`` (sorted paths, file order), parsed."""
    for path in sorted(Path(root).rglob("*.list")):
        for line in path.read_text().splitlines():
            line = line.strip()
            if line and not line.startswith("#"):
                yield cl.parse_case(line)


def census(root):
    groups, foreign = defaultdict(list), 0
    for c in walk(root):
        if c["op"] not in SERVED:
            foreign += 1
            continue
        groups[group_key(c)].append(c)
    table = {}
    for key in sorted(groups):
        toks = sorted(tokens_of(c) for c in groups[key])
        table[key] = {"records": len(toks), "batch_sizes": len({c["batch_size"] for c in groups[key]}),
                      "tokens": [toks[0], toks[len(toks) // 2], toks[-1]]}
    return {"served_records": sum(v["records"] for v in table.values()), "foreign_records": foreign, "groups": table}, groups


def pick(groups):
    lines = []
    for n, key in enumerate(sorted(groups)):
        recs = groups[key]
        h = int(hashlib.sha256(key.encode()).hexdigest(), 16)
        chosen = [max(recs, key=lambda c: (c["batch_size"], tokens_of(c))), recs[h % len(recs)]]
        if recs[0]["phase"] == "P":
            chosen.append(min(recs, key=tokens_of))
            if n % 4 == 0:
                chosen.append(max(recs, key=tokens_of))
        seen = set()
        for c in chosen:
            if c["_raw_line"] not in seen:
                seen.add(c["_raw_line"])
                lines.append(c["_raw_line"])
    return lines


def main():
    root = sys.argv[1]
    table, groups = census(root)
    (HERE / "corpus_census.json").write_text(json.dumps(table, indent=1, sort_keys=True) + "\n")
    lines = pick(groups)
    (HERE / "corpus_sample.list").write_text(
        "# A few records per shape group of the reference's case corpus; made by make_caselist_sample.py.\n"
        + "\n".join(lines) + "\n")
    print(table["served_records"], "records in", len(groups), "groups ->", len(lines), "sampled")


if __name__ == "__main__":
    main()
