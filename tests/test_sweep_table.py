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


def _write(path, backend, times, dtype="float32", reduce="sum", algo="-", mode="w"):
    with open(path, mode) as f:
        f.write("NCCL version 2.27\n")  # the tool's stdout may carry other lines
        for (op, nbytes), t in times.items():
            f.write(json.dumps({"backend": backend, "op": op, "dtype": dtype, "reduce": reduce, "bytes": nbytes,
                                "time_us": t, "busbw_gbs": nbytes / t / 1e3, "algo": algo, "ok": True}) + "\n")


def test_table_has_one_row_per_case_and_ratios_against_the_first_run(tmp_path):
    st = _module()
    a, b = tmp_path / "a.json", tmp_path / "b.json"
    _write(a, "nccl", {("all_reduce", 1024): 20.0, ("all_reduce", 1 << 30): 2600.0})
    _write(b, "nvl", {("all_reduce", 1024): 10.0, ("all_reduce", 1 << 30): 2860.0, ("all_gather", 4096): 5.0})
    text = st.table([f"reference={a}", f"ours={b}:nvl"])
    rows = text.splitlines()
    assert rows[0].startswith("| op | dtype | reduce | bytes | reference us / GB/s | ours us / GB/s | algorithm | reference / ours")
    assert "| all_reduce | float32 | sum | 1 KiB | 20.0 / 0 | 10.0 / 0 | - | 2.00x |" in text
    assert "| all_reduce | float32 | sum | 1 GiB |" in text and "0.91x" in text
    assert "| all_gather | float32 | sum | 4 KiB | - | 5.0 / 1 | - | - |" in text
    assert st.human(3 * (1 << 20)) == "3 MiB" and st.human(1000) == "1000 B"


def test_summary_spans_dtypes_and_reduce_ops(tmp_path):
    st = _module()
    a, b = tmp_path / "a.json", tmp_path / "b.json"
    _write(a, "nccl", {("all_reduce", 1024): 20.0})
    _write(a, "nccl", {("all_reduce", 1024): 30.0}, dtype="int8", reduce="max", mode="a")
    _write(b, "nvl", {("all_reduce", 1024): 10.0}, algo="flagged-words")
    _write(b, "nvl", {("all_reduce", 1024): 10.0}, dtype="int8", reduce="max", algo="flagged-words", mode="a")
    text = st.summary([f"reference={a}", f"nvl={b}"])
    assert "| all_reduce | 1 KiB |" in text and "2.00x .. 3.00x" in text and "| 2 | 0 |" in text
