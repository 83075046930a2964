"""The stand-in for Ray that the reference arm of the benchmark uses when Ray is not installed
(``baseline/ray_shim``): actors placed in another process, named actors, fail-fast ``ray.get``, ``ray.wait``,
timeouts and ``ray.kill``, exercised with two CPU processes."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys, time
    sys.path.insert(0, os.path.join(sys.argv[3], "baseline", "ray_shim"))
    import ray
    rank, world = int(sys.argv[1]), 2
    rt = ray._core.start(rank, world, sys.argv[2])
    ray._core.set_placement(lambda kind, target, a, k, o: a[0] if getattr(target, "__name__", "") == "Echo" else None)

    @ray.remote
    class Echo:
        def __init__(self, where):
            self.where, self.seen = where, []
        def pid(self):
            return (self.where, os.getpid())
        def append(self, obj):
            obj.append(1)          # arguments arrive as copies: the caller's list must stay empty
            self.seen.append(len(obj))
            return self.seen
        def boom(self):
            raise KeyError("x")
        def slow(self):
            time.sleep(1.0)
            return "late"

    @ray.remote
    class Store:
        def __init__(self, v):
            self.v = v
        def get(self):
            return self.v

    @ray.remote
    def where_am_i(tag):
        return (tag, os.getpid())

    if rank == 1:
        rt.serve_until_shutdown()
        os._exit(0)
    a0, a1 = Echo.remote(0), Echo.remote(1)
    r = ray.get([a0.pid.remote(), a1.pid.remote()])
    assert r[0][1] == os.getpid() and r[1][1] != os.getpid(), r
    mine = []
    assert ray.get(a0.append.remote(mine)) == [1] and mine == []       # copy semantics, also in-process
    assert ray.get(a0.append.remote(mine)) == [1, 1]                    # calls of one actor run in order
    s = Store.options(name="s", lifetime="detached").remote(7)
    assert ray.get(ray.get_actor("s").get.remote()) == 7
    again = Store.options(name="s", get_if_exists=True).remote(9)
    assert ray.get(again.get.remote()) == 7
    try:
        ray.get_actor("nope")
        raise SystemExit("lookup of an unknown name must fail")
    except ValueError:
        pass
    try:
        ray.get([a0.slow.remote(), a1.boom.remote()])                   # fails fast on the second reference
        raise SystemExit("ray.get must re-raise the actor's exception")
    except KeyError:
        pass
    done, pending = ray.wait([a1.pid.remote()], num_returns=1)
    assert len(done) == 1 and not pending
    try:
        ray.get(a1.slow.remote(), timeout=0.05)
        raise SystemExit("timeout expected")
    except ray.exceptions.GetTimeoutError:
        pass
    assert ray.get(where_am_i.remote("t"))[0] == "t"
    ray.kill(s)
    try:
        ray.get_actor("s")
        raise SystemExit("killed actors lose their name")
    except ValueError:
        pass
    rt.shutdown_all()
    print("shim ok")
''')


def test_ray_stand_in_with_two_processes(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    rdv = tmp_path / "rdv"
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(rdv), ROOT], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in (1, 0)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "shim ok" in outs[1]
