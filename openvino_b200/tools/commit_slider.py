"""commit_slider: walk a list of commits with a build command and an application command and find where a behaviour
changes (first failing commit by output pattern, first commit whose benchmark number degrades, or every break).

    python -m openvino_b200.tools.commit_slider -c config.json [-s start..end]

Configuration (JSON):
  gitPath        repository to walk (default: current directory)
  commitList     {"getCommitListCmd": "git log a..b --boundary --pretty=%h"} or {"explicitList": [...]}  (oldest last, as git prints)
  buildCmd       shell command run in the work tree after every checkout (optional)
  appCmd         shell command whose output is examined
  runConfig      {"mode": "checkOutput", "stopPattern": "<regex>"}                      commit is bad when the pattern matches
                 {"mode": "benchmark", "metricPattern": "<regex with one group>", "threshold": 0.1, "higherIsBetter": true}
                 "traversal": "firstFailedVersion" | "firstFixedVersion" | "allBreaks"
Every commit is checked out into a scratch work tree (``git worktree``), so the repository's own checkout is untouched.
Role of tools/commit_slider/commit_slider.py with its modes (utils/modes.py) and traversals (utils/traversal.py).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
from typing import Callable, Dict, List, Optional


def _sh(cmd: str, cwd: str, check: bool = True) -> str:
    r = subprocess.run(cmd, shell=True, cwd=cwd, capture_output=True, text=True)
    if check and r.returncode != 0:
        raise RuntimeError("command failed (%d): %s\n%s" % (r.returncode, cmd, r.stderr[-2000:]))
    return r.stdout + r.stderr


class Slider:
    def __init__(self, cfg: dict, log: Callable[[str], None] = print):
        self.cfg = cfg
        self.git = os.path.abspath(cfg.get("gitPath", "."))
        self.log = log
        self.cache: Dict[str, dict] = {}
        self.tree: Optional[str] = None

    # ---- commits, oldest first
    def commits(self, interval: Optional[str] = None) -> List[str]:
        cl = self.cfg.get("commitList", {})
        if "explicitList" in cl:
            lst = list(cl["explicitList"])
        else:
            cmd = cl.get("getCommitListCmd") or "git log %s --boundary --pretty=%%h" % (interval or "")
            if interval and "getCommitListCmd" in cl:
                cmd = cl["getCommitListCmd"].replace("{interval}", interval)
            lst = [l.strip() for l in _sh(cmd, self.git).splitlines() if l.strip()]
        lst = [c.lstrip("-").strip() for c in lst]
        return list(reversed(lst))            # git prints newest first

    # ---- one commit
    def run_commit(self, commit: str) -> dict:
        if commit in self.cache:
            return self.cache[commit]
        if self.tree is None:
            self.tree = tempfile.mkdtemp(prefix="commit_slider_")
            _sh("git worktree add --detach %s %s" % (self.tree, commit), self.git)
        else:
            _sh("git checkout --detach -f %s" % commit, self.tree)
        if self.cfg.get("buildCmd"):
            _sh(self.cfg["buildCmd"], self.tree)
        out = _sh(self.cfg["appCmd"], self.tree, check=False)
        res = {"commit": commit, "output": out}
        rc = self.cfg.get("runConfig", {})
        if rc.get("mode", "checkOutput") == "benchmark":
            m = re.search(rc["metricPattern"], out)
            res["metric"] = float(m.group(1)) if m else None
        else:
            res["bad"] = re.search(rc.get("stopPattern", "error|fail"), out) is not None
        self.cache[commit] = res
        self.log("  %s -> %s" % (commit, res.get("metric", res.get("bad"))))
        return res

    def close(self) -> None:
        if self.tree is not None:
            _sh("git worktree remove --force %s" % self.tree, self.git, check=False)
            shutil.rmtree(self.tree, ignore_errors=True)
            self.tree = None

    # ---- is `commit` different (worse) than the reference commit `base`?
    def differs(self, base: dict, cur: dict) -> bool:
        rc = self.cfg.get("runConfig", {})
        if rc.get("mode", "checkOutput") == "benchmark":
            a, b = base.get("metric"), cur.get("metric")
            if a is None or b is None:
                return a != b
            thr = float(rc.get("threshold", 0.1))
            return (b < a * (1 - thr)) if rc.get("higherIsBetter", True) else (b > a * (1 + thr))
        return bool(cur["bad"]) != bool(base["bad"])

    # ---- traversals
    def first_break(self, commits: List[str]) -> Optional[str]:
        """Binary search: the first commit that differs from the oldest one (assumes one break in the interval)."""
        base = self.run_commit(commits[0])
        if not self.differs(base, self.run_commit(commits[-1])):
            return None
        lo, hi = 0, len(commits) - 1              # commits[lo] like base, commits[hi] differs
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self.differs(base, self.run_commit(commits[mid])):
                hi = mid
            else:
                lo = mid
        return commits[hi]

    def all_breaks(self, commits: List[str]) -> List[str]:
        out = []

        def rec(lo: int, hi: int):
            if hi <= lo or not self.differs(self.run_commit(commits[lo]), self.run_commit(commits[hi])):
                return
            if hi - lo == 1:
                out.append(commits[hi])
                return
            mid = (lo + hi) // 2
            rec(lo, mid)
            rec(mid, hi)
        rec(0, len(commits) - 1)
        return out

    def run(self, interval: Optional[str] = None) -> dict:
        commits = self.commits(interval)
        if len(commits) < 2:
            raise RuntimeError("need at least two commits, got %r" % commits)
        trav = self.cfg.get("runConfig", {}).get("traversal", "firstFailedVersion")
        try:
            if trav == "allBreaks":
                return {"traversal": trav, "breaks": self.all_breaks(commits), "checked": len(self.cache)}
            return {"traversal": trav, "break": self.first_break(commits), "checked": len(self.cache)}
        finally:
            self.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("-c", "--config", required=True)
    ap.add_argument("-s", "--interval", default=None, help="commit interval start..end")
    args = ap.parse_args(argv)
    with open(args.config) as f:
        cfg = json.load(f)
    res = Slider(cfg).run(args.interval)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
