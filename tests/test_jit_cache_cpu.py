"""The in-tree kernel image cache: keys follow the generated source AND the hand-written headers
(a header edit never reuses an old image), hits refresh the entry, prune() evicts least recently
used images first.  The compiler is replaced by a stub: no nvcc run, no GPU."""
import os
import time

from evt_ae_b200 import jit


def _use_tmp_cache(tmp_path, monkeypatch):
    monkeypatch.setattr(jit, "CACHE_DIR", str(tmp_path))
    calls = []

    class Done:
        returncode, stdout, stderr = 0, "", "ptxas info: stub"

    def fake_run(cmd, capture_output=True, text=True):
        calls.append(cmd)
        out = cmd[cmd.index("-o") + 1]
        with open(out, "wb") as f:
            f.write(b"\0" * 1000)
        return Done()
    monkeypatch.setattr(jit.subprocess, "run", fake_run)
    return calls


def test_key_covers_source_and_headers(tmp_path, monkeypatch):
    calls = _use_tmp_cache(tmp_path, monkeypatch)
    a = jit.compile_cubin("// kernel A")
    assert jit.compile_cubin("// kernel A") == a and len(calls) == 1          # hit: no second build
    b = jit.compile_cubin("// kernel B")
    assert b != a and len(calls) == 2
    monkeypatch.setattr(jit, "_header_digest", "another-version-of-the-headers")
    a2 = jit.compile_cubin("// kernel A")
    assert a2 != a and len(calls) == 3                                          # same source, new headers: rebuilt
    assert os.path.exists(a) and os.path.exists(a + ".cu") and os.path.exists(a + ".log")


def test_prune_evicts_least_recently_used(tmp_path, monkeypatch):
    _use_tmp_cache(tmp_path, monkeypatch)
    paths = []
    for i in range(5):
        p = jit.compile_cubin(f"// kernel {i}")
        os.utime(p, (time.time() - 1000 + i, time.time() - 1000 + i))
        paths.append(p)
    jit.compile_cubin("// kernel 0")                   # a hit refreshes kernel 0
    per = jit.cache_entries()[0][2]
    removed = jit.prune(3 * per)
    assert removed == 2
    assert os.path.exists(paths[0]) and not os.path.exists(paths[1]) and not os.path.exists(paths[2])
    assert not os.path.exists(paths[1] + ".cu") and os.path.exists(paths[4])
    assert jit.prune(10 ** 9) == 0
