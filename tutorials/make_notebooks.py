"""Write a Jupyter notebook next to every tutorial script.

    python tutorials/make_notebooks.py [--check]

The tutorials are kept as Python scripts in the "percent" format (``# %%`` opens a code cell, ``# %% [markdown]`` a
text cell whose lines are comments), which diff well and run under ``pytest``.  This script turns each of them into
``tutorials/notebooks/<name>.ipynb`` (nbformat 4, no outputs) for readers who prefer a notebook; ``--check`` only
verifies that the notebooks on disk are what the scripts produce (used by ``tests/test_tutorials.py``).
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "notebooks")


def cells_of(source: str):
    """``[(kind, [lines])]`` with kind "code" or "markdown"; text before the first marker is a code cell."""
    cells, kind, lines = [], "code", []
    for line in source.splitlines():
        if line.startswith("# %%"):
            if any(x.strip() for x in lines):
                cells.append((kind, lines))
            kind = "markdown" if "[markdown]" in line else "code"
            lines = []
        else:
            lines.append(line)
    if any(x.strip() for x in lines):
        cells.append((kind, lines))
    return cells


def notebook_of(source: str) -> dict:
    out = []
    for kind, lines in cells_of(source):
        while lines and not lines[0].strip():
            lines = lines[1:]
        while lines and not lines[-1].strip():
            lines = lines[:-1]
        if kind == "markdown":
            text = [x[2:] if x.startswith("# ") else x.lstrip("#") for x in lines]
            out.append({"cell_type": "markdown", "metadata": {}, "source": [t + "\n" for t in text[:-1]] + text[-1:]})
        else:
            # a notebook has no __file__: the scripts' "run from a source checkout" line becomes a relative path
            lines = ['sys.path.insert(0, os.path.abspath(os.path.join("..", "..")))   # repository root, from tutorials/notebooks'
                     if "sys.path.insert" in x and "__file__" in x else x for x in lines]
            out.append({"cell_type": "code", "execution_count": None, "metadata": {}, "outputs": [],
                        "source": [t + "\n" for t in lines[:-1]] + lines[-1:]})
    return {"cells": out, "metadata": {"kernelspec": {"display_name": "Python 3", "language": "python", "name": "python3"},
                                       "language_info": {"name": "python"}},
            "nbformat": 4, "nbformat_minor": 5}


def scripts():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".py") and f != os.path.basename(__file__))


def render(name: str) -> str:
    with open(os.path.join(HERE, name), encoding="utf-8") as f:
        return json.dumps(notebook_of(f.read()), indent=1, ensure_ascii=False) + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    os.makedirs(OUT, exist_ok=True)
    stale = []
    for name in scripts():
        target = os.path.join(OUT, name[:-3] + ".ipynb")
        text = render(name)
        if args.check:
            if not os.path.exists(target) or open(target, encoding="utf-8").read() != text:
                stale.append(os.path.basename(target))
        else:
            with open(target, "w", encoding="utf-8") as f:
                f.write(text)
            print("wrote", os.path.relpath(target, os.path.dirname(HERE)))
    if stale:
        print("out of date:", ", ".join(stale))
        sys.exit(1)


if __name__ == "__main__":
    main()
