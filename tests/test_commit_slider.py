"""commit_slider on a scratch git repository: finds the commit where the output pattern / the benchmark number changes."""
import subprocess

from openvino_b200.tools.commit_slider import Slider


def _repo(tmp_path, values):
    r = tmp_path / "repo"
    r.mkdir()
    run = lambda *a: subprocess.run(a, cwd=r, check=True, capture_output=True, text=True).stdout.strip()
    run("git", "init", "-q")
    run("git", "config", "user.email", "t@example.com")
    run("git", "config", "user.name", "t")
    hashes = []
    for i, v in enumerate(values):
        (r / "app.py").write_text("# revision %d\nprint('fps: %s')\nprint(%r)\n" % (i, v[0], v[1]))
        run("git", "add", "-A")
        run("git", "commit", "-q", "-m", "c%d" % i)
        hashes.append(run("git", "rev-parse", "--short", "HEAD"))
    return str(r), hashes


def test_first_failed_commit_by_output(tmp_path):
    vals = [(100, "ok")] * 5 + [(100, "error: wrong blob")] * 4
    repo, hashes = _repo(tmp_path, vals)
    cfg = {"gitPath": repo, "commitList": {"explicitList": list(reversed(hashes))}, "appCmd": "python app.py",
           "runConfig": {"mode": "checkOutput", "stopPattern": "error", "traversal": "firstFailedVersion"}}
    res = Slider(cfg, log=lambda s: None).run()
    assert res["break"] == hashes[5] and res["checked"] <= 5


def test_benchmark_degradations(tmp_path):
    vals = [(100, "x")] * 3 + [(80, "x")] * 3 + [(60, "x")] * 2
    repo, hashes = _repo(tmp_path, vals)
    cfg = {"gitPath": repo, "commitList": {"getCommitListCmd": "git log --pretty=%h"}, "appCmd": "python app.py",
           "runConfig": {"mode": "benchmark", "metricPattern": r"fps: ([0-9.]+)", "threshold": 0.1, "traversal": "allBreaks"}}
    res = Slider(cfg, log=lambda s: None).run()
    assert res["breaks"] == [hashes[3], hashes[6]]
