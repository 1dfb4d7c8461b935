"""bench/sweep_table.py: JSON lines of the benchmark tool -> markdown comparison table."""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _module():
    spec = importlib.util.spec_from_file_location("sweep_table", os.path.join(ROOT, "bench", "sweep_table.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _write(path, backend, times):
    with open(path, "w") as f:
        f.write("NCCL version 2.27\n")  # the tool's stdout may carry other lines
        for (op, nbytes), t in times.items():
            f.write(json.dumps({"backend": backend, "op": op, "bytes": nbytes, "time_us": t,
                                "busbw_gbs": nbytes / t / 1e3, "ok": True}) + "\n")


def test_table_has_one_row_per_case_and_ratios_against_the_first_run(tmp_path):
    st = _module()
    a, b = tmp_path / "a.json", tmp_path / "b.json"
    _write(a, "nccl", {("all_reduce", 1024): 20.0, ("all_reduce", 1 << 30): 2600.0})
    _write(b, "nvl", {("all_reduce", 1024): 10.0, ("all_reduce", 1 << 30): 2860.0, ("all_gather", 4096): 5.0})
    text = st.table([f"reference={a}", f"ours={b}:nvl"])
    rows = text.splitlines()
    assert rows[0].startswith("| op | bytes | reference us / GB/s | ours us / GB/s | reference / ours")
    assert "| all_reduce | 1 KiB | 20.0 / 0 | 10.0 / 0 | 2.00x |" in text
    assert "| all_reduce | 1 GiB |" in text and "0.91x" in text
    assert "| all_gather | 4 KiB | - | 5.0 / 1 | - |" in text
    assert st.human(3 * (1 << 20)) == "3 MiB" and st.human(1000) == "1000 B"
