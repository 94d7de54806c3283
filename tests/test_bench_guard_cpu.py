"""bench.py's guard over the extra legs of a multi-GPU run: a rank that does not come back from
a leg must not hold the run until a collective library's own time-out.  The guard is a timer on
every rank; when it runs out rank 0 prints the JSON line as it stands and the process ends with
status 0.  Checked here with a child process whose "leg" sleeps past the deadline."""
import json
import subprocess
import sys
import textwrap

CHILD = textwrap.dedent('''
    import sys, time, json
    sys.path.insert(0, %r)
    import bench
    line = {"metric": "m", "value": 1.0}
    guard = bench.ExtrasGuard(int(sys.argv[2]), line, sys.stdout, seconds=1.0)
    if sys.argv[1] == "hang":
        time.sleep(60)          # a leg that never returns
        print("not reached")
    else:
        line["extra"] = 2       # a leg that ends in time
        assert guard.finish()
        print(json.dumps(line))
''')


def run_child(mode, rank):
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return subprocess.run([sys.executable, "-c", CHILD % root, mode, str(rank)],
                          capture_output=True, text=True, timeout=30)


def test_a_leg_that_hangs_ends_with_the_headline_line():
    r = run_child("hang", 0)
    assert r.returncode == 0
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["metric"] == "m" and line["value"] == 1.0 and "extras_abandoned" in line


def test_other_ranks_leave_silently():
    r = run_child("hang", 3)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_legs_that_finish_print_the_full_line_once():
    r = run_child("ok", 0)
    assert r.returncode == 0
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["extra"] == 2
