"""Run ruff and report only findings on lines that differ from a base revision.

    python .github/scripts/ruff_changed_lines.py origin/main

Lets the lint job gate new code without demanding that the whole tree is reformatted first (the reference's CI does
the same with its own script, ``.github/scripts/ruff_diff.py``).  Exit status 1 when a changed line has a finding.
"""

from __future__ import annotations

import json
import re
import subprocess
import sys


def changed_lines(base: str) -> dict[str, set[int]]:
    diff = subprocess.run(["git", "diff", "--unified=0", base, "--", "*.py"], capture_output=True, text=True, check=True).stdout
    out: dict[str, set[int]] = {}
    current = None
    for line in diff.splitlines():
        if line.startswith("+++ b/"):
            current = line[6:]
            out.setdefault(current, set())
        elif line.startswith("@@") and current is not None:
            m = re.search(r"\+(\d+)(?:,(\d+))?", line)
            start, count = int(m.group(1)), int(m.group(2) or 1)
            out[current].update(range(start, start + count))
    return {f: ls for f, ls in out.items() if ls}


def main() -> int:
    base = sys.argv[1] if len(sys.argv) > 1 else "origin/main"
    touched = changed_lines(base)
    if not touched:
        print("no python lines changed")
        return 0
    res = subprocess.run(["ruff", "check", "--output-format", "json", "--line-length", "130", *touched], capture_output=True, text=True)
    findings = json.loads(res.stdout or "[]")
    hits = []
    for f in findings:
        path = f["filename"]
        rel = next((t for t in touched if path.endswith(t)), None)
        if rel and f["location"]["row"] in touched[rel]:
            hits.append(f"{rel}:{f['location']['row']}: {f['code']} {f['message']}")
    print("\n".join(hits) if hits else f"ruff: no findings on {sum(map(len, touched.values()))} changed lines")
    return 1 if hits else 0


if __name__ == "__main__":
    sys.exit(main())
