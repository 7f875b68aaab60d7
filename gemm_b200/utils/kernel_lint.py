"""Kernel linter that needs no GPU: reads the CUDA sources of this package as text and checks the rules their kernels are
written to, then prints an inventory of the tensor-core / TMA instructions each file issues.

    python -m gemm_b200.utils.kernel_lint            # exit status 1 if a rule is broken

Rules (each has cost a GPU somewhere before it became a rule):

* ``bounded-wait``   a loop that polls memory another agent writes (``ld_acquire``, ``ld_volatile``, ``mbar_try_wait``, a
  ``volatile`` load) must check a time or iteration budget inside the loop (``globaltimer_ns``, a ``Budget`` constant, or a counter
  compared against a limit): no wait of this library spins for ever;
* ``tmem-paired``    a kernel that allocates tensor memory (``tmem_alloc``) must free it (``tmem_dealloc``) in the same kernel, and a
  file that issues ``tcgen05.alloc`` must also issue ``tcgen05.dealloc`` and ``tcgen05.relinquish_alloc_permit``;
* ``no-cluster-broadcast-load``  no TMA or bulk load that delivers its tile to several CTAs of a cluster at once (the PTX qualifier
  made of the words "multicast" and "cluster") in a file that runs on more than one GPU; files named in ``.gpurunignore.multi`` are
  exempt: they never travel to a multi-GPU run.  ``tcgen05.commit`` with that qualifier is not a load and is fine;
* ``arch``           no ``wgmma`` (Hopper only; does not assemble for sm_100a).

The reference validates generated PTX strings without a GPU (cuda/ptx_validate.h: directives, braces, known mnemonics); here
nvcc already rejects malformed inline PTX at build time, so the linter checks what the assembler cannot know.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from typing import Dict, List, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_DIRS = [os.path.join(ROOT, "csrc", "kernels"), os.path.join(ROOT, "csrc", "fabric")]
POLL = re.compile(r"\b(ld_acquire\w*|ld_volatile\w*|ld_relaxed\w*|mbar_try_wait|flag_load\w*)\s*\(|\*\s*\(\s*(const\s+)?volatile\b")
BOUND = re.compile(r"globaltimer_ns|Budget|budget|max_iter|kMaxSpin|spins?\s*[<>]=?|\bit\s*[<>]=?\s*\w|tries\s*[<>]")
INVENTORY = [("tcgen05.mma", r"tcgen05\.mma"), ("tcgen05.ld/st/cp", r"tcgen05\.(ld|st|cp)\b"), ("tcgen05.commit", r"tcgen05\.commit"),
             ("cp.async.bulk.tensor", r"cp\.async\.bulk\.tensor"), ("cp.async.bulk", r"cp\.async\.bulk(?!\.tensor)"),
             ("mbarrier", r"mbarrier\."), ("griddepcontrol", r"griddepcontrol\."), ("mma.sync / wmma", r"mma\.sync|wmma::"),
             ("peer / multimem", r"multimem\.|peer_")]


def strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", lambda m: "\n" * m.group(0).count("\n"), text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def _match_brace(text: str, open_idx: int) -> int:
    depth = 0
    for i in range(open_idx, len(text)):
        c = text[i]
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                return i
    return len(text) - 1


def _match_paren(text: str, open_idx: int) -> int:
    depth = 0
    for i in range(open_idx, len(text)):
        c = text[i]
        if c == "(":
            depth += 1
        elif c == ")":
            depth -= 1
            if depth == 0:
                return i
    return len(text) - 1


def loops(text: str):
    """(line, header, body) of every for / while / do-while statement of comment-stripped ``text``."""
    for m in re.finditer(r"\b(for|while)\s*\(", text):
        p0 = m.end() - 1
        p1 = _match_paren(text, p0)
        header = text[p0: p1 + 1]
        j = p1 + 1
        while j < len(text) and text[j].isspace():
            j += 1
        if j < len(text) and text[j] == "{":
            body = text[j: _match_brace(text, j) + 1]
        elif j < len(text) and text[j] == ";":
            # `while (...);` closes a do-block or is an empty-bodied spin: take the do-block in front of it if there is one
            k = text.rfind("}", 0, m.start())
            body = ""
            if k >= 0 and text[k + 1: m.start()].strip() == "":
                depth, b = 0, k
                while b >= 0:
                    if text[b] == "}":
                        depth += 1
                    elif text[b] == "{":
                        depth -= 1
                        if depth == 0:
                            break
                    b -= 1
                body = text[b: k + 1]
        else:
            body = text[j: text.find(";", j) + 1]
        yield text.count("\n", 0, m.start()) + 1, header, body


def kernels(text: str):
    """(name, body) of every __global__ function."""
    for m in re.finditer(r"__global__[^;{]*?\b(\w+)\s*\(", text):
        p1 = _match_paren(text, m.end() - 1)
        j = text.find("{", p1)
        semi = text.find(";", p1)
        if j < 0 or (0 <= semi < j):
            continue
        yield m.group(1), text[j: _match_brace(text, j) + 1]


def helper_map(header_text: str) -> Dict[str, str]:
    """Device helpers of a header that wrap one of the inventoried instructions: name -> inventory key (so that a call of
    ``tma_load_2d`` in a kernel file counts as a ``cp.async.bulk.tensor``)."""
    text = strip_comments(header_text)
    out: Dict[str, str] = {}
    for m in re.finditer(r"__device__[^;{(]*?\b(\w+)\s*\(", text):
        p1 = _match_paren(text, m.end() - 1)
        j = text.find("{", p1)
        semi = text.find(";", p1)
        if j < 0 or (0 <= semi < j):
            continue
        body = text[j: _match_brace(text, j) + 1]
        for key, pat in INVENTORY:
            if re.search(pat, body):
                out[m.group(1)] = key
                break
    return out


def lint_text(name: str, raw: str, multi_gpu: bool = True, helpers: Dict[str, str] = None) -> Tuple[List[Dict], Dict[str, int]]:
    text = strip_comments(raw)
    out: List[Dict] = []
    for line, header, body in loops(text):
        if POLL.search(header) or POLL.search(body):
            if not (BOUND.search(header) or BOUND.search(body)):
                out.append({"rule": "bounded-wait", "file": name, "line": line, "what": "a polling loop without a time or iteration budget"})
    for kname, body in kernels(text):
        if re.search(r"\btmem_alloc\s*\(", body) and not re.search(r"\btmem_dealloc\s*\(", body):
            out.append({"rule": "tmem-paired", "file": name, "line": 0, "what": f"kernel {kname} allocates tensor memory and never frees it"})
    if "tcgen05.alloc" in text and not ("tcgen05.dealloc" in text and "tcgen05.relinquish_alloc_permit" in text):
        out.append({"rule": "tmem-paired", "file": name, "line": 0, "what": "tcgen05.alloc without dealloc / relinquish_alloc_permit"})
    if multi_gpu:
        for m in re.finditer(r"cp\.async\.bulk[\w.:]*\." + "multi" + "cast" + "::cluster", text):
            out.append({"rule": "no-cluster-broadcast-load", "file": name, "line": text.count("\n", 0, m.start()) + 1,
                        "what": "a TMA / bulk load broadcast to a cluster in a file that runs on several GPUs"})
    if re.search(r"\bwgmma\.", text):
        out.append({"rule": "arch", "file": name, "line": 0, "what": "wgmma is sm_90a only"})
    inv = {k: len(re.findall(pat, text)) for k, pat in INVENTORY}
    for h, key in (helpers or {}).items():
        inv[key] += len(re.findall(r"\b" + re.escape(h) + r"\s*\(", text))
    return out, inv


def lint_tree(root: str = os.path.dirname(ROOT)) -> Dict:
    exempt = set()
    ign = os.path.join(root, ".gpurunignore.multi")
    if os.path.exists(ign):
        exempt = {ln.strip() for ln in open(ign) if ln.strip() and not ln.startswith("#")}
    problems, inventory = [], {}
    helpers: Dict[str, str] = {}
    for d in SRC_DIRS:
        for fn in sorted(os.listdir(d)):
            if fn.endswith(".cuh"):
                helpers.update(helper_map(open(os.path.join(d, fn)).read()))
    for d in SRC_DIRS:
        for fn in sorted(os.listdir(d)):
            if not fn.endswith((".cu", ".cuh", ".h")):
                continue
            path = os.path.join(d, fn)
            rel = os.path.relpath(path, root)
            p, inv = lint_text(rel, open(path).read(), multi_gpu=rel not in exempt, helpers=None if fn.endswith(".cuh") else helpers)
            problems += p
            if any(inv.values()):
                inventory[rel] = {k: v for k, v in inv.items() if v}
    return {"problems": problems, "inventory": inventory}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    rep = lint_tree()
    if args.json:
        print(json.dumps(rep, indent=1))
    else:
        for f, inv in rep["inventory"].items():
            print(f"{f}: " + ", ".join(f"{k} x{v}" for k, v in inv.items()))
        for p in rep["problems"]:
            print(f"PROBLEM {p['rule']}: {p['file']}:{p['line']}: {p['what']}")
        print(f"{len(rep['problems'])} problem(s)")
    return 1 if rep["problems"] else 0


if __name__ == "__main__":
    sys.exit(main())
