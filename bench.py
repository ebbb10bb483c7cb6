"""Benchmark of the PCVR inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" scores one per-GPU batch of synthetic samples with the OneTrans model.  The default
workload is the full-scale configuration: per GPU 8 192 samples, 64 sparse fields with
1 000 001 x 128 bf16 tables (Zipf 1.1 ids), one behaviour sequence of Zipf ids with lengths uniform
in [128, 1024] padded to 1024, 8 blocks, d_model 512, 8 heads, hidden_mult 4; weights from seed 0,
identical on every rank; rank r draws its batch from data seed r (weak scaling).  Rank 0 prints ONE
JSON line:

* ``value``       samples/s of the whole job with the batches already resident in HBM (four batches per rank
                  rotate through the timed steps; a pass of K steps is repeated until about two seconds have been
                  timed and the median pass is reported);
* ``e2e``         the same through the public call (``score_stream``) with HOST (pinned) inputs: H2D copy of the
                  batch, forward, NCCL gather of the scores (N > 1), D2H read of the scores, every step;
* ``roofline``    algorithmic work / CUDA-event time of the dominant hand-written kernel inside the
                  timed steps, against the measured peaks in MEASURED_PEAKS.json; ``kernels`` lists every
                  timed launch group (library launches included) and ``step_accounting`` the share of the
                  step they cover;
* ``cpu_baseline`` the reference's own ``PCVROneTrans`` (compiled form under ``oracle/_ref``, kind
                  ``"reference"``; the vectorised port ``oracle/torch_cpu.py``, kind ``"port"``, where that
                  archive is missing) on a bounded sample of the same batch, all host threads (rank 0, N = 1
                  only), with the score parity of ``--parity-rows`` rows against the GPU outside the timed region.

``--impl reference`` times only that CPU arm (same config, bounded sample per step) and says in its line what ran.
``--workload norm|attention|gather|ffn`` run the standalone operator sweeps (also what the ncu
profiles under profiles/ were captured from); they print one JSON line per case.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from taac_2026_b200 import _lib, ops  # noqa: E402
from taac_2026_b200.inputs import OneTransSpec, compact_model_input, synthetic_batch  # noqa: E402
from taac_2026_b200.onetrans import OneTransInference, random_state_dict, score_stream  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def full_scale_spec() -> OneTransSpec:
    return OneTransSpec(
        user_int_specs=[(1_000_000, i, 1) for i in range(48)],
        item_int_specs=[(1_000_000, i, 1) for i in range(16)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [1_000_000]},
        d_model=512, emb_dim=128, num_blocks=8, num_heads=8, hidden_mult=4, seq_top_k=1024,
        user_ns_tokens=5, item_ns_tokens=2,
    )


def small_spec() -> OneTransSpec:
    """The baseline-sized configuration (batch 512, 32 fields x 100 001 x 64, L 256, d 128, 4 heads, 2 blocks)."""
    return OneTransSpec(
        user_int_specs=[(100_000, i, 1) for i in range(24)],
        item_int_specs=[(100_000, i, 1) for i in range(8)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [1_000_000]},
        d_model=128, emb_dim=64, num_blocks=2, num_heads=4, hidden_mult=4, seq_top_k=256,
        user_ns_tokens=5, item_ns_tokens=2,
    )


WORKLOADS = {
    "full": dict(spec=full_scale_spec, batch=8192, seq_len=1024, min_len=128, field_exp=1.1, seq_exp=1.1, micro=8192,
                 name="OneTrans full scale: 8192 samples/GPU, 64 fields x 1000001 x 128 bf16, L<=1024, d512 h8 x8 layers"),
    "small": dict(spec=small_spec, batch=512, seq_len=256, min_len=16, field_exp=1.2, seq_exp=1.1, micro=512,
                  name="OneTrans baseline size: 512 samples, 32 fields x 100001 x 64, L<=256, d128 h4 x2 layers"),
}


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc: subprocess.Popen | None = None
        self.lines: list[str] = []
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


# ------------------------------------------------------------------------------------------------
# roofline accounting from the per-launch timing records
# ------------------------------------------------------------------------------------------------
def attention_flops(meta: dict) -> float:
    """4 * D * H * (visible query-key pairs): valid queries x visible keys only."""
    heads, dim, lk, lq = meta["heads"], meta["dim"], meta["lk"], meta["lq"]
    if meta.get("cu_rows") is not None:
        rows = (meta["cu_rows"][1:] - meta["cu_rows"][:-1]).double()
        if meta.get("cu_rows_q") is not None:   # the last `qn` rows of every sample are the queries
            qn = (meta["cu_rows_q"][1:] - meta["cu_rows_q"][:-1]).double()
            pairs = (qn * (rows - qn) + qn * (qn + 1) / 2).sum().item() if meta["causal"] else (qn * rows).sum().item()
            return 4.0 * dim * heads * pairs
        pairs = (rows * (rows + 1) / 2).sum().item() if meta["causal"] else (rows * rows).sum().item()
        return 4.0 * dim * heads * pairs
    if meta.get("key_valid") is not None:
        kv = meta["key_valid"].double()
        if meta["causal"]:
            pairs = (torch.cumsum(kv, dim=1) * kv).sum().item()
        else:
            pairs = (kv.sum(dim=1) * lq).sum().item()
        return 4.0 * dim * heads * pairs
    batch = meta["batch"]
    ns_start = min(meta["ns_start"], lk)
    ns = lk - ns_start
    if meta["seq_len"] is None:
        ell = torch.full((batch,), float(ns_start), dtype=torch.float64)
    else:
        ell = meta["seq_len"].double().clamp(min=0, max=ns_start).cpu()
    if meta["causal"]:
        pairs = ell * (ell + 1) / 2 + ns * ell + ns * (ns + 1) / 2
        if not meta["self_rows"]:  # padded queries still attend (no self fallback): keys <= q that are valid
            pairs = pairs + (ns_start - ell) * ell
    else:
        q_rows = (ell + ns) if meta["self_rows"] else torch.full_like(ell, float(lq))
        pairs = q_rows * (ell + ns)
    return 4.0 * dim * heads * pairs.sum().item()


def launch_work(name: str, meta: dict) -> tuple[str, float]:
    """-> (bound, algorithmic bytes or flops) of one recorded launch."""
    if name.startswith("attention"):
        row_bytes = meta["heads"] * meta["dim"] * meta.get("esize", 2)
        if meta.get("cu_rows_q") is not None:
            # a few queries per sample against all of its keys: every K / V row is read once and used by a handful
            # of queries (about 17 FLOP per byte on the full workload), so HBM bounds this launch, not the tensor pipe
            k_rows = float(meta["cu_rows"][-1].item())
            q_rows = float(meta["cu_rows_q"][-1].item())
            return "hbm", 2.0 * row_bytes * (k_rows + q_rows)
        if name == "attention_small":
            # samples of at most 32 rows (the 9 non-sequence tokens of a sample): a few hundred FLOP per row against
            # one read of q, k, v and one write of o, so the stream over the rows is what bounds it
            rows = float(meta["cu_rows"][-1].item()) if meta.get("cu_rows") is not None else float(meta["batch"] * meta["lk"])
            return "hbm", 4.0 * row_bytes * rows
        return "tensor", attention_flops(meta)
    if name == "bias_act_rows":     # in place: read + write of the matrix
        return "hbm", 2.0 * meta["rows"] * meta["cols"] * meta["esize"]
    if name == "add_gathered_rows":  # in place: read + write of the matrix + the ids; the small tables are served by the L2
        return "hbm", 2.0 * meta["rows"] * meta["dim"] * meta["esize"] + 8.0 * meta["tables"] * meta["rows"]
    if name == "token_tail":
        # one read and one write of the matrix, the write of the (possibly compacted) first output, the ids and, with
        # row selection, one int32 per row; the small tables are served by the L2
        row_bytes = meta["cols"] * meta["esize"]
        select = 4.0 * meta["rows"] if meta["rows_out"] != meta["rows"] else 0.0
        return "hbm", row_bytes * (2.0 * meta["rows"] + meta["rows_out"]) + 8.0 * meta["tables"] * meta["rows"] + select
    if name == "token_project":
        # fused tokenizer: every DISTINCT table row in once (repeats are served by the L2), the full-height normalised
        # rows and the kept token rows out, the feature ids, the two ids of the added rows and the int32 destination
        ids = meta["ids"]
        row_bytes = meta["k"] // ids.shape[0] * 2
        distinct = sum(int(torch.unique(ids[f]).numel()) for f in range(ids.shape[0]))
        out_bytes = 2.0 * meta["cols"] * (meta["rows"] + meta["rows_out"])
        return "hbm", float(distinct * row_bytes) + out_bytes + 8.0 * ids.numel() + 20.0 * meta["rows"]
    if name == "scatter_rows":
        return "hbm", 3.0 * meta["rows"] * meta["dim"] * meta["esize"] + 8.0 * meta["rows"]
    if name in ("rms_norm", "layer_norm"):
        extra = meta["cols"] * meta["esize"] * (2 if name == "layer_norm" else 1)
        return "hbm", 2.0 * meta["rows"] * meta["cols"] * meta["esize"] + extra
    if name in ("gemm_bf16", "cublas_linear"):
        return "tensor", 2.0 * meta.get("groups", 1) * meta["m"] * meta["n"] * meta["k"]
    if name.startswith("fp8_gemm") or name.startswith("mx_gemm"):
        return "tensor_fp8", 2.0 * meta["m"] * meta["n"] * meta["k"]
    if name == "quant_act":
        return "hbm", meta["rows"] * meta["cols"] * 3.0 + meta["rows"] * (meta["cols"] // 128) * 4.0
    if name in ("fields_bag_mean", "sequence_gather", "gather_rows"):
        ids = meta["ids"]
        valid = int(torch.unique(ids[ids != 0]).numel())   # distinct rows: repeats are served by the L2
        row_bytes = meta["dim"] * meta["esize"]
        out_rows = ids.numel()
        if name == "fields_bag_mean":
            out_rows = ids.shape[0] * meta["n_fields"]
        return "hbm", float(valid * row_bytes + out_rows * row_bytes + ids.numel() * ids.element_size())
    return "hbm", 0.0


def summarise_kernels(records: list, peaks: dict, peak_kind: str, steps: int, fp8_peak: float | None,
                      pass_ms: float) -> tuple[dict | None, dict, dict]:
    """Group the timing records by operator -> (roofline of the dominant one, per-op table, accounting).

    Every launch of this library and every library GEMM call site left in the engine carries an event pair.
    What lies between one record's end and the next record's start on the stream is the rest of the step: ATen
    index / copy / reduce kernels and the gaps in which the GPU waits for the host.  It is measured the same
    way (event to event) and reported as one line, so that the table sums to the step it was taken from."""
    table: dict[str, dict] = {}
    between_ms = 0.0
    prev_end = None
    for name, meta, start, end in records:
        bound, work = launch_work(name, meta)
        entry = table.setdefault(name, {"launches": 0, "ms": 0.0, "work": 0.0, "bound": bound})
        entry["launches"] += 1
        entry["ms"] += start.elapsed_time(end)
        entry["work"] += work
        if prev_end is not None:
            between_ms += max(prev_end.elapsed_time(start), 0.0)
        prev_end = end
    if not table:
        return None, {}, {}
    bf16_peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 0.0)))
    for entry in table.values():
        seconds = entry["ms"] * 1e-3
        if entry["bound"] in ("tensor", "tensor_fp8"):
            entry["achieved"] = entry["work"] / seconds / 1e12 if seconds > 0 else 0.0
            entry["unit"] = "TFLOP/s"
            entry["peak"] = bf16_peak
            if entry["bound"] == "tensor_fp8":
                # the e4m3 library GEMM measured in this run when there is one, else twice the measured bf16 figure
                entry["peak"] = float(fp8_peak) if fp8_peak else 2.0 * bf16_peak
                entry["bound"] = "tensor"
        else:
            entry["achieved"] = entry["work"] / seconds / 1e9 if seconds > 0 else 0.0
            entry["unit"] = "GB/s"
            entry["peak"] = float(peaks.get("hbm_gbs", 0.0))
        entry["frac"] = entry["achieved"] / entry["peak"] if entry["peak"] else None
    top_name = max(table, key=lambda n: table[n]["ms"])
    top = table[top_name]
    traffic = None
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        try:
            per_unit = json.loads(traffic_file.read_text()).get(top_name)
            if per_unit is not None:
                traffic = per_unit["dram_bytes_per_unit_work"] * top["work"] / max(top["launches"], 1)
        except Exception:
            traffic = None
    roofline = {
        "kernel": top_name, "bound": top["bound"], "achieved": round(top["achieved"], 3), "peak": top["peak"],
        "unit": top["unit"], "frac": None if top["frac"] is None else round(top["frac"], 4), "traffic": traffic,
        "peak_source": f"{peak_kind} (MEASURED_PEAKS.json)" if peak_kind == "measured" else "fallback",
        "launches": top["launches"], "avg_launch_ms": round(top["ms"] / max(top["launches"], 1), 4),
        "own_kernel": not top_name.startswith("cublas"),
    }
    per_op = {
        n: {"launches": e["launches"], "ms": round(e["ms"], 3), "ms_per_step": round(e["ms"] / steps, 4),
            "achieved": round(e["achieved"], 2), "unit": e["unit"], "frac": None if e["frac"] is None else round(e["frac"], 4)}
        for n, e in sorted(table.items(), key=lambda kv: -kv[1]["ms"])
    }
    recorded = sum(e["ms"] for e in table.values())
    library = sum(e["ms"] for n, e in table.items() if n.startswith("cublas"))
    accounting = {
        "pass_ms_per_step": round(pass_ms / steps, 3),
        "own_kernels_ms_per_step": round((recorded - library) / steps, 3),
        "library_gemm_ms_per_step": round(library / steps, 3),
        "aten_glue_and_gaps_ms_per_step": round(between_ms / steps, 3),
        "accounted_frac": round((recorded + between_ms) / pass_ms, 4) if pass_ms > 0 else None,
        "note": "event pairs around every launch of this library and every library GEMM call site; the glue line is "
                "the stream time between consecutive records (ATen index / copy / reduce kernels and host-bound gaps)",
    }
    return roofline, per_op, accounting


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own PCVROneTrans where it can be imported, else the vectorised port
# ------------------------------------------------------------------------------------------------
def host_memory_available() -> int:
    """Bytes this process may still allocate on the host: MemAvailable, capped by the cgroup limit."""
    avail = 1 << 62
    try:
        for line in Path("/proc/meminfo").read_text().splitlines():
            if line.startswith("MemAvailable:"):
                avail = int(line.split()[1]) * 1024
    except OSError:
        pass
    for name in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            text = Path(name).read_text().strip()
            if text.isdigit():
                used = 0
                for cur in ("/sys/fs/cgroup/memory.current", "/sys/fs/cgroup/memory/memory.usage_in_bytes"):
                    try:
                        used = int(Path(cur).read_text().strip())
                        break
                    except (OSError, ValueError):
                        continue
                avail = min(avail, int(text) - used)
        except OSError:
            continue
    return avail


class CpuArm:
    """The CPU implementation of the path that the GPU numbers are put beside.

    kind "reference": the unmodified ``PCVROneTrans.predict`` of the reference (experiments/onetrans/model.py:354-359,
    torch backend, fp32), imported through ``oracle/ref_runtime.py``; its parameters are the GPU model's, widened to
    fp32.  kind "port": ``oracle/torch_cpu.py`` (same library calls, tables kept in their stored type), used where the
    reference cannot be imported or its fp32 tables do not fit the host's memory."""

    def __init__(self, spec: OneTransSpec, sd: dict[str, torch.Tensor], *, prefer: str = "reference") -> None:
        self.spec = spec
        self.spec_dict = spec.as_dict()
        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        self.kind, self.why_port = "port", ""
        self.model = None
        if prefer == "reference":
            try:
                from oracle import ref_runtime

                if not ref_runtime.available():
                    raise RuntimeError("no reference checkout and no oracle/_ref on this machine")
                need = sum(t.numel() for t in sd.values()) * 4
                have = host_memory_available()
                if have < 1.6 * need:
                    raise RuntimeError(f"fp32 parameters need {need / 2**30:.0f} GiB, host offers {have / 2**30:.0f} GiB")
                sd32 = {name: t.to(device="cpu", dtype=torch.float32) for name, t in sd.items()}
                self.model = ref_runtime.build_model(self.spec_dict, state_dict=sd32, meta_init=True)
                self._predict = lambda batch: ref_runtime.predict(self.model, batch)
                self.kind = "reference"
                self.form = ref_runtime.import_reference()
            except Exception as error:  # noqa: BLE001 - any failure falls back to the port, with the reason kept
                self.why_port = f"{type(error).__name__}: {error}"
        if self.kind == "port":
            from oracle import torch_cpu

            sd_cpu = cpu_state_dict(sd)
            self._predict = lambda batch: torch_cpu.predict(sd_cpu, self.spec_dict, batch)

    def predict(self, batch):
        with torch.no_grad():
            return self._predict(batch)

    def describe(self) -> dict:
        out = {"kind": self.kind, "cores": torch.get_num_threads()}
        if self.kind == "reference":
            out["implementation"] = f"reference PCVROneTrans.predict, torch backend, fp32 ({self.form} form)"
        else:
            out["implementation"] = "oracle/torch_cpu.py (vectorised port of the reference torch path)"
            if self.why_port:
                out["reference_not_used_because"] = self.why_port
        return out


def cpu_state_dict(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Weights on the host for the port: tables keep their storage type (rows are widened after the gather), the
    dense layers are fp32."""
    out = {}
    for name, t in sd.items():
        is_table = ".embeddings." in name or ".compressed_embeddings." in name or name.endswith("time_embedding.weight")
        out[name] = t.cpu() if is_table else t.float().cpu()
    return out


def time_cpu_arm(arm: CpuArm, batch_cpu, *, steps: int, warmup: int, budget_s: float, max_rows: int) -> dict:
    """`warmup` + `steps` passes of the CPU arm, each over the same bounded sample of the batch; the sample is sized
    from a probe so that all passes together take about `budget_s` seconds."""
    rows = min(8, batch_cpu.batch_size)
    t0 = time.perf_counter()
    arm.predict(batch_cpu.slice(0, rows))  # first call: allocator and thread-pool warm-up, not a measurement
    t0 = time.perf_counter()
    arm.predict(batch_cpu.slice(0, rows))
    per_row = max((time.perf_counter() - t0) / rows, 1e-6)
    passes = max(1, steps) + max(0, warmup)
    sample = int(max(rows, min(batch_cpu.batch_size, max_rows, budget_s / passes / per_row)))
    sample_batch = batch_cpu.slice(0, sample)
    logits = None
    for _ in range(max(0, warmup)):
        arm.predict(sample_batch)
    times = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        logits, _ = arm.predict(sample_batch)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {
        "value": round(sample / med, 2), "unit": "samples/s", **arm.describe(),
        "sample": f"first {sample} rows of the rank-0 batch per pass, {len(times)} timed + {max(0, warmup)} warm-up passes, median",
        "seconds": round(med, 4), "seconds_min_max": [round(min(times), 4), round(max(times), 4)],
        "_rows": sample, "_logits": logits,
    }


def score_parity(arm: CpuArm, model, host_batch, rows: int, chunk: int = 256) -> dict:
    """Scores of the first `rows` samples on the GPU (the benchmarked precision) against the CPU arm, outside any
    timed region: largest score difference and the AUC of both score vectors on labels drawn from the CPU logits
    (standardised, so that the AUC is well away from 0.5)."""
    from oracle import reference_ops as R

    want_logits = []
    for lo in range(0, rows, chunk):
        want_logits.append(arm.predict(host_batch.slice(lo, min(lo + chunk, rows)))[0].reshape(-1).float())
    want_logits = torch.cat(want_logits)
    want = torch.sigmoid(want_logits)
    got = model.scores(host_batch.slice(0, rows).to(model.device)).cpu().reshape(-1)
    model.raise_if_incomplete()
    z = (want_logits - want_logits.mean()) / want_logits.std().clamp_min(1e-6)
    labels = (torch.rand(rows, generator=torch.Generator().manual_seed(2)) < torch.sigmoid(2.0 * z)).numpy()
    auc_cpu, auc_gpu = R.binary_auc(labels, want.numpy()), R.binary_auc(labels, got.numpy())
    return {
        "parity_rows": rows, "max_abs_score_diff_vs_gpu": round(float((want - got).abs().max()), 6),
        "auc_cpu": round(auc_cpu, 6), "auc_gpu": round(auc_gpu, 6), "auc_abs_diff": round(abs(auc_cpu - auc_gpu), 7),
        "auc_equal_to_4_decimals": round(auc_cpu, 4) == round(auc_gpu, 4),
    }


def run_parity_stages(args) -> None:
    """Score parity by precision stage, outside any timed region: the first ``--parity-rows`` samples of the full-scale
    batch are scored by the CPU arm in fp32 (the yardstick) and by the GPU engine in four precisions, from the fp32
    parity mode to the benchmarked one; where the reference can be imported, its own model also runs on the GPU under
    bf16 autocast (its serving precision, `runtime_autocast_context`, runtime/execution.py:54-60), which shows how far
    16-bit serving moves the reference itself.  One JSON line per stage: largest score difference and both AUCs."""
    from oracle import reference_ops as R

    wl = WORKLOADS["full" if args.workload == "parity" else args.workload]
    spec: OneTransSpec = wl["spec"]()
    rows = args.parity_rows if args.parity_rows > 256 else 8192
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    batch = synthetic_batch(spec, rows, seq_len=wl["seq_len"], min_len=wl["min_len"], seed=0,
                            field_exponent=wl["field_exp"], seq_exponent=wl["seq_exp"])
    sd = random_state_dict(spec, seed=0, device=dev, dtype=torch.bfloat16)
    arm = CpuArm(spec, sd)
    chunk = 256
    t0 = time.perf_counter()
    want_logits = torch.cat([arm.predict(batch.slice(lo, min(lo + chunk, rows)))[0].reshape(-1).float()
                             for lo in range(0, rows, chunk)])
    cpu_seconds = time.perf_counter() - t0
    want = torch.sigmoid(want_logits)
    z = (want_logits - want_logits.mean()) / want_logits.std().clamp_min(1e-6)
    labels = (torch.rand(rows, generator=torch.Generator().manual_seed(2)) < torch.sigmoid(2.0 * z)).numpy()
    auc_cpu = R.binary_auc(labels, want.numpy())
    base = {"metric": "score_parity_by_stage", "rows": rows, "yardstick": arm.describe(), "yardstick_seconds": round(cpu_seconds, 1),
            "auc_yardstick": round(auc_cpu, 6), "config": {"workload": wl["name"]}}

    # the AUC difference of one label draw is a handful of swapped pairs; 32 further draws show its spread
    draws = [(torch.rand(rows, generator=torch.Generator().manual_seed(100 + i)) < torch.sigmoid(2.0 * z)).numpy() for i in range(32)]
    auc_cpu_draws = [R.binary_auc(d, want.numpy()) for d in draws]

    def report(stage: str, got: torch.Tensor, **extra) -> None:
        got = got.detach().float().cpu().reshape(-1)
        auc = R.binary_auc(labels, got.numpy())
        deltas = [abs(R.binary_auc(d, got.numpy()) - a) for d, a in zip(draws, auc_cpu_draws)]
        extra = {**extra, "auc_abs_diff_32_label_draws": {"mean": round(float(sum(deltas) / len(deltas)), 7), "max": round(float(max(deltas)), 7)},
                 "rank_correlation_with_yardstick": round(float(torch.corrcoef(torch.stack([want.argsort().argsort().float(), got.argsort().argsort().float()]))[0, 1]), 8)}
        print(json.dumps({**base, "stage": stage, "max_abs_score_diff": round(float((want - got).abs().max()), 7),
                          "mean_abs_score_diff": round(float((want - got).abs().mean()), 8), "auc": round(auc, 6),
                          "auc_abs_diff": round(abs(auc - auc_cpu), 7),
                          "auc_equal_to_4_decimals": round(auc, 4) == round(auc_cpu, 4), **extra}), flush=True)

    dev_batch = batch.to(dev)
    if arm.kind == "reference":
        # the reference's own module on the GPU, torch backend, fp32 parameters, bf16 autocast
        from oracle import ref_runtime

        sd32 = {name: t.float() for name, t in sd.items()}
        ref_gpu = ref_runtime.build_model(spec.as_dict(), state_dict=sd32, meta_init=True)
        outs = []
        with torch.autocast("cuda", dtype=torch.bfloat16):
            for lo in range(0, rows, chunk):
                outs.append(ref_runtime.predict(ref_gpu, dev_batch.slice(lo, min(lo + chunk, rows)))[0].reshape(-1).float())
        report("reference model on the GPU, torch backend, bf16 autocast", torch.sigmoid(torch.cat(outs)))
        outs = []
        for lo in range(0, rows, chunk):
            outs.append(ref_runtime.predict(ref_gpu, dev_batch.slice(lo, min(lo + chunk, rows)))[0].reshape(-1).float())
        report("reference model on the GPU, torch backend, fp32 (TF32 off)", torch.sigmoid(torch.cat(outs)))
        del ref_gpu, sd32, outs
        torch.cuda.empty_cache()
    stages = [("this engine: fp32 dense layers and attention", torch.float32, "bf16"),
              ("this engine: bf16, bf16 FFN", torch.bfloat16, "bf16"),
              ("this engine: bf16, FP8 FFN with GEMM 1 in bf16", torch.bfloat16, "fp8_precise"),
              ("this engine: bf16, FP8 FFN with power-of-two scales inside the block-scaled MMA", torch.bfloat16, "fp8_mx"),
              ("this engine: bf16, FP8 FFN (benchmarked precision)", torch.bfloat16, "fp8")]
    for name, dtype, ffn in stages:
        weights = sd if dtype == torch.bfloat16 else {k: v.float() for k, v in sd.items()}
        model = OneTransInference(weights, spec, device=dev, dtype=dtype, ffn=ffn)
        got = torch.cat([model.scores(dev_batch.slice(lo, min(lo + 2048, rows))).reshape(-1) for lo in range(0, rows, 2048)])
        model.raise_if_incomplete()
        report(name, got)
        del model, weights, got
        torch.cuda.empty_cache()


# ------------------------------------------------------------------------------------------------
# main benchmark
# ------------------------------------------------------------------------------------------------
def run_e2e(args) -> None:
    import torch.distributed as dist

    from taac_2026_b200.dist import gather_scores

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.workload]
    spec: OneTransSpec = wl["spec"]()
    batch_size = args.batch or wl["batch"]
    peaks, peak_kind = load_peaks()

    def make_batch(seed: int):
        return synthetic_batch(spec, batch_size, seq_len=wl["seq_len"], min_len=wl["min_len"], seed=seed,
                               field_exponent=wl["field_exp"], seq_exponent=wl["seq_exp"])

    if args.impl == "reference":
        # The CPU arm alone, on rank 0: every step is one pass of the reference's torch path over a bounded sample of
        # the workload's batch, on all host threads.  The other ranks have nothing to do.
        if rank != 0:
            return
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        sd = random_state_dict(spec, seed=0, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
        arm = CpuArm(spec, sd)
        del sd
        if dev == "cuda":
            torch.cuda.empty_cache()
        res = time_cpu_arm(arm, make_batch(0).slice(0, min(batch_size, 512)), steps=args.steps, warmup=args.warmup,
                           budget_s=60.0, max_rows=256)
        rows = res.pop("_rows")
        res.pop("_logits")
        line = {
            "impl": "reference", "metric": "pcvr_infer_samples_per_s", "value": res["value"], "unit": "samples/s",
            "n_gpus": args.gpus, "device": "cpu", "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(res["seconds"] * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "per_gpu_batch": batch_size, "rows_per_step": rows,
                       "note": "runs on the host CPU of rank 0 only, whatever --gpus says: every step is one pass of "
                               "the reference torch path over the first rows_per_step samples of the batch"},
            "cpu_baseline": res,
            "e2e": {"value": res["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for the cuda backend)")
    torch.cuda.set_device(local_rank)
    if not ops.cuda_available():
        raise RuntimeError("libtb200.so is missing or the device is not sm_100")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)

    sd = random_state_dict(spec, seed=0, device=dev, dtype=torch.bfloat16)
    ffn_mode = args.ffn if spec.d_model % 256 == 0 else "bf16"
    model = OneTransInference(sd, spec, device=dev, dtype=torch.bfloat16, ffn=ffn_mode, packed=not args.padded,
                              select_early=not args.late_select, attention_kernel=args.kernel,
                              fused_tokenizer=args.fused_tokenizer)
    # Distinct batches rotate through both arms (rank r draws seeds r, r + 1000, ...), so that no step meets the ids,
    # lengths or duplicate pattern of the step before it.
    n_rot = max(1, args.rotate)
    host_batches = [make_batch(rank + 1000 * i).pin_memory() for i in range(n_rot)]
    dev_batches = [b.to(dev) for b in host_batches]
    # What the end-to-end arm copies every step.  "compact32": the sequences as 32-bit valid prefixes, written by the
    # library's host packer (the job of the data loader's batch converter, outside the timed region like the rest of
    # batch construction; its cost per batch is reported) and expanded to the padded int64 record by one kernel on the
    # device inside the timed region.  "padded64": the reference's padded int64 record as it is.
    stream_batches, pack_ms = host_batches, None
    if args.host_format == "compact32":
        try:
            t0 = time.perf_counter()
            stream_batches = [compact_model_input(b, threads=4, pin=True) for b in host_batches]
            pack_ms = (time.perf_counter() - t0) * 1e3 / n_rot
        except OverflowError:
            args.host_format = "padded64 (a value did not fit the 32-bit format)"
    micro = args.micro_batch or wl["micro"]
    host_scores = torch.empty(world * batch_size if world > 1 else batch_size, dtype=torch.float32).pin_memory()
    counter = {"resident": 0, "e2e": 0}

    def step_resident() -> torch.Tensor:
        batch = dev_batches[counter["resident"] % n_rot]
        counter["resident"] += 1
        return gather_scores(model.scores(batch, micro_batch=micro))

    def run_stream(steps: int) -> None:
        """`steps` batches from pinned host memory through the public serving loop (`score_stream`): every step
        copies its inputs to the device (on a side stream, under the previous step's kernels), gathers the scores
        of all ranks and reads them back to the host."""
        first = counter["e2e"]
        counter["e2e"] += steps
        stream = (stream_batches[(first + i) % n_rot] for i in range(steps))
        for scores in score_stream(model, stream, micro_batch=micro, prepare_ahead=not args.no_prepare_ahead):
            host_scores.copy_(gather_scores(scores), non_blocking=True)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int, sink: list | None) -> float:
        barrier()
        ops.set_kernel_timing(sink)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        ops.set_kernel_timing(None)
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    if args.profile:
        # for a profiler: few launches before the interesting ones, no timing events, no second arm
        for _ in range(args.warmup):
            step_resident()
        barrier()
        for _ in range(args.steps):
            step_resident()
        barrier()
        if rank == 0:
            print(json.dumps({"profile_run": True, "steps": args.steps, "warmup": args.warmup,
                              "note": "not a measurement: no warm-up floor, no timing"}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    warmup = max(args.warmup, 3)
    for _ in range(max(warmup, n_rot)):
        step_resident()
    run_stream(min(2, n_rot))
    model.raise_if_incomplete()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # Timed regions.  A pass is exactly K steps between barrier + synchronize on both sides (max over ranks); passes
    # are repeated until the arm has been timed for about two seconds, and the MEDIAN pass is the one reported.
    #   resident: inputs already in HBM                            -> `value`
    #   e2e:      pinned host batches through score_stream          -> `e2e`
    #   recorded: resident steps with an event pair per launch     -> `roofline`, `kernels` (its own time is reported)
    launches_before = _lib.launch_count()
    first_ms = timed(step_resident, args.steps, None)
    launches = _lib.launch_count() - launches_before
    n_pass = max(3, min(25, int(args.min_timed_s * 1e3 / max(first_ms, 1e-3)) + 1))
    resident_passes = [first_ms] + [timed(step_resident, args.steps, None) for _ in range(n_pass - 1)]
    ms_total = statistics.median(resident_passes)
    e2e_passes = [timed(lambda: run_stream(args.steps), 1, None) for _ in range(n_pass)]
    ms_e2e = statistics.median(e2e_passes)
    # the accounting pass: event pairs around every launch.  One throw-away pass first, so that the recorded one does
    # not pay for the switch back from the serving loop's stream (its memory pool) or for the first event objects
    timed(step_resident, args.steps, [])
    records: list = []
    ms_recorded = timed(step_resident, args.steps, records)
    # the same resident steps in the reference's order of operations (every block for every row, then the
    # pyramid's row selection), for comparison with `value`
    ms_ref_order = None
    if model.packed and model.select_early and not args.no_reference_order:
        model.select_early = False
        for _ in range(2):
            step_resident()
        ms_ref_order = timed(step_resident, args.steps, None)
        model.select_early = True
    clocks = sampler.stop() if rank == 0 else {}
    model.raise_if_incomplete()

    # Multi-GPU result check (untimed): rank 0 scores rank 1's first batch itself and compares it bit for bit with
    # rank 1's slice of the gathered vector (same kernels, same inputs, no atomics on the path).
    multi_gpu_check = None
    if world > 1:
        gathered = gather_scores(model.scores(dev_batches[0], micro_batch=micro))
        if rank == 0:
            own = model.scores(make_batch(1).to(dev), micro_batch=micro)
            same = bool(torch.equal(gathered[batch_size:2 * batch_size], own))
            multi_gpu_check = {"rank1_slice_bit_identical_to_rank0_recompute": same, "rows": batch_size,
                               "gathered_rows": int(gathered.numel())}
            if not same:
                print("WARNING: gathered scores of rank 1 differ from rank 0's recomputation", file=sys.stderr, flush=True)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    fp8_peak = measure_fp8_peak() if ffn_mode.startswith("fp8") else None
    roofline, per_op, accounting = summarise_kernels(records, peaks, peak_kind, args.steps, fp8_peak, ms_recorded)
    if args.launch_log:
        with open(args.launch_log, "w") as fh:
            for name, meta, ev0, ev1 in records:
                bound, work = launch_work(name, meta)
                shape = {k: v for k, v in meta.items() if isinstance(v, (int, float, bool, str))}
                fh.write(json.dumps({"name": name, "ms": round(ev0.elapsed_time(ev1), 4), "bound": bound, "work": work, **shape}) + "\n")
    del records
    total = batch_size * world
    value = total * args.steps / (ms_total * 1e-3)
    e2e_value = total * args.steps / (ms_e2e * 1e-3)
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        arm = CpuArm(spec, sd)
        cpu = time_cpu_arm(arm, host_batches[0], steps=3, warmup=1, budget_s=20.0, max_rows=256)
        cpu.pop("_rows"), cpu.pop("_logits")
        # the same rows on the GPU, in the benchmarked precision: a full-scale check of scores and AUC
        cpu.update(score_parity(arm, model, host_batches[0], min(batch_size, max(args.parity_rows, 256))))
        del arm
    extra = {}
    if world == 1 and args.workload == "full" and not args.no_op_lines:
        del dev_batches
        torch.cuda.empty_cache()
        extra["c3_attention"] = attention_lines(peaks, peak_kind, batch=256, steps=3)
        extra["c4_ffn"] = ffn_lines(peaks, peak_kind, rows=262144, steps=3, fp8_peak=fp8_peak)
    line = {
        "metric": "pcvr_infer_samples_per_s", "value": round(value, 2), "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_total / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 activations, e4m3 FFN GEMMs" if ffn_mode.startswith("fp8") else "bf16", "data": "synthetic",
        "config": {
            "workload": wl["name"], "per_gpu_batch": batch_size, "global_batch": total, "micro_batch": micro,
            "ffn": ffn_mode, "layout": "padded" if args.padded else "packed valid tokens",
            "pyramid_row_selection": "after the block (reference order)" if (args.late_select or args.padded) else "keys/values for all rows; queries, attention and the row-wise half of each block for the rows the pyramid keeps",
            "parallelism": f"batch-sharded x{world}, scores all_gather", "weights": "seed 0, bf16",
            "batches": f"{n_rot} distinct batches per rank in rotation",
            "l2": "activations and tables (>= 16 GB) are far larger than the 126 MB L2",
        },
        "clocks": clocks,
        "timing": {"passes": n_pass, "steps_per_pass": args.steps, "reported": "median pass",
                   "timed_region_s": round(sum(resident_passes) * 1e-3, 3),
                   "ms_per_step_passes": [round(m / args.steps, 3) for m in resident_passes]},
        "e2e": {"value": round(e2e_value, 2), "unit": "samples/s",
                "h2d_bytes_per_step": stream_batches[0].nbytes(), "host_format": args.host_format,
                "padded_int64_record_bytes": host_batches[0].nbytes(),
                "host_pack_ms_per_batch": None if pack_ms is None else round(pack_ms, 2),
                "d2h_bytes_per_step": host_scores.numel() * 4, "ms_per_step": round(ms_e2e / args.steps, 3),
                "passes_ms_per_step": [round(m / args.steps, 3) for m in e2e_passes], "reported": "median pass",
                "timed_region_s": round(sum(e2e_passes) * 1e-3, 3)},
        "gpu_launches": launches,
        "reference_order": None if ms_ref_order is None else {
            "value": round(total * args.steps / (ms_ref_order * 1e-3), 2), "unit": "samples/s",
            "ms_per_step": round(ms_ref_order / args.steps, 3),
            "note": "same steps with the pyramid's row selection after each whole block, as the reference orders it",
        },
        "roofline": roofline,
        "kernels": per_op,
        "step_accounting": accounting,
        "fp8_library_gemm_tflops": None if fp8_peak is None else round(fp8_peak, 1),
        "multi_gpu_check": multi_gpu_check,
        "cpu_baseline": cpu,
        **extra,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# operator sweeps
# ------------------------------------------------------------------------------------------------
def graph_time(fn, buffers: list, reps: int) -> float:
    """Average ms of fn(buffer) over a CUDA graph that walks `buffers` (total size > L2) `reps` times."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for buf in buffers:
            fn(buf)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for buf in buffers:
                fn(buf)
        graph.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
    return start.elapsed_time(end) / (reps * len(buffers))


def run_norm_sweep(args) -> None:
    """65 536 x {128, 256, 512, 1024} bf16, 1 % outlier rows; buffers rotate through > 400 MB."""
    peaks, peak_kind = load_peaks()
    rows = args.rows or 65536
    for cols in ([args.cols] if args.cols else [128, 256, 512, 1024]):
        g = torch.Generator(device="cuda").manual_seed(0)
        n_buf = max(2, int(400e6 // (rows * cols * 2)) + 1) if not args.cols else 6
        bufs = []
        for _ in range(n_buf):
            x = torch.randn(rows, cols, generator=g, device="cuda")
            x[torch.randperm(rows, device="cuda")[: rows // 100]] *= 50.0
            bufs.append(x.bfloat16())
        w = (1 + 0.02 * torch.randn(cols, generator=g, device="cuda")).bfloat16()
        b = (0.02 * torch.randn(cols, generator=g, device="cuda")).bfloat16()
        for name, fn in (("rms_norm", lambda x: ops.rms_norm(x, w, 1e-6)), ("layer_norm", lambda x: ops.layer_norm(x, w, b, 1e-6))):
            if args.kind and args.kind != name:
                continue
            ms = graph_time(fn, bufs, args.steps)
            nbytes = 2.0 * rows * cols * 2 + cols * 2 * (2 if name == "layer_norm" else 1)
            gbs = nbytes / ms / 1e6
            print(json.dumps({
                "metric": f"{name}_fwd_GBps", "value": round(gbs, 1), "unit": "GB/s", "config": {"workload": f"{rows}x{cols} bf16"},
                "us_per_launch": round(ms * 1e3, 2),
                "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peak_kind},
            }), flush=True)


def run_norm_backward_sweep(args) -> None:
    """RMSNorm / LayerNorm backward on 65 536 x {128, 256, 512, 1024} bf16 rows: x and dy in, dx out
    (3 * rows * cols * 2 bytes of algorithmic HBM traffic); buffers rotate through > 400 MB."""
    peaks, peak_kind = load_peaks()
    rows = args.rows or 65536
    for cols in ([args.cols] if args.cols else [128, 256, 512, 1024]):
        g = torch.Generator(device="cuda").manual_seed(0)
        n_buf = max(2, int(400e6 // (rows * cols * 4)) + 1)
        bufs = [(torch.randn(rows, cols, generator=g, device="cuda").bfloat16(), torch.randn(rows, cols, generator=g, device="cuda").bfloat16())
                for _ in range(n_buf)]
        w = (1 + 0.02 * torch.randn(cols, generator=g, device="cuda")).bfloat16()
        b = (0.02 * torch.randn(cols, generator=g, device="cuda")).bfloat16()
        for name, fn in (("rms_norm_bwd", lambda p: ops.rms_norm_backward(p[0], w, p[1], 1e-6)),
                         ("layer_norm_bwd", lambda p: ops.layer_norm_backward(p[0], w, b, p[1], 1e-6))):
            ms = graph_time(fn, bufs, args.steps)      # a CUDA graph over the rotating buffers: device time, not host time
            gbs = 3.0 * rows * cols * 2 / ms / 1e6
            print(json.dumps({
                "metric": f"{name}_GBps", "value": round(gbs, 1), "unit": "GB/s", "config": {"workload": f"{rows}x{cols} bf16"},
                "us_per_call": round(ms * 1e3, 2), "note": "two launches per call (row kernel + reduction of the partial sums)",
                "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peak_kind},
            }), flush=True)


def run_token_tail_sweep(args) -> None:
    """token_tail on 262 144 x 512 bf16 rows: LayerNorm(SiLU(x)) + two gathered table rows -> tokens, RMSNorm -> normed.
    Algorithmic HBM bytes: one read and two writes of the matrix plus the ids (the 1025- and 64-row tables stay in L2)."""
    peaks, peak_kind = load_peaks()
    rows, cols = args.rows or 262144, args.cols or 512
    g = torch.Generator(device="cuda").manual_seed(0)
    bufs = [torch.randn(rows, cols, generator=g, device="cuda").bfloat16() for _ in range(3)]
    w1, b1, w2 = ((1 + 0.02 * torch.randn(cols, generator=g, device="cuda")).bfloat16() for _ in range(3))
    pos = torch.randn(1025, cols, generator=g, device="cuda").bfloat16()
    tim = torch.randn(64, cols, generator=g, device="cuda").bfloat16()
    ip = torch.randint(0, 1025, (rows,), generator=g, device="cuda")
    it = torch.randint(0, 64, (rows,), generator=g, device="cuda")
    ms = graph_time(lambda x: ops.token_tail(x, w1, b1, tim, it, pos, ip, w2), bufs, args.steps)
    nbytes = 3.0 * rows * cols * 2 + 16.0 * rows
    gbs = nbytes / ms / 1e6
    print(json.dumps({
        "metric": "token_tail_GBps", "value": round(gbs, 1), "unit": "GB/s", "config": {"workload": f"{rows}x{cols} bf16, two tables"},
        "us_per_launch": round(ms * 1e3, 2),
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peak_kind},
    }), flush=True)


def attention_lines(peaks: dict, peak_kind: str, *, batch: int, steps: int, kernel: int = 0, seed: int = 0) -> list[dict]:
    """Varlen padded-mask attention: `batch` samples (a slice of the 2048), 8 heads, head_dim 64, L 1024, lengths
    uniform in [32, 1024]; non-causal + key padding and causal + key padding.  FLOPs count valid queries x
    visible keys only."""
    B, H, L, D = batch, 8, 1024, 64
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(B, H, L, D, generator=g, device="cuda").div_(8).bfloat16() for _ in range(3))
    lens = torch.randint(32, 1025, (B,), generator=g, device="cuda", dtype=torch.int32)
    out = []
    for causal in (False, True):
        fn = lambda: ops.varlen_attention(q, k, v, seq_len=lens, causal=causal, padded_query_self=causal, kernel=kernel)  # noqa: E731
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / steps
        ell = lens.double().cpu()
        pairs = (ell * (ell + 1) / 2).sum().item() if causal else (ell * L).sum().item()
        valid_pairs = (ell * (ell + 1) / 2).sum().item() if causal else (ell * ell).sum().item()
        tf = 4.0 * D * H * valid_pairs / ms / 1e9
        peak = peaks["bf16_tflops"]
        out.append({
            "metric": "attention_fwd_TFLOPs", "value": round(tf, 1), "unit": "TFLOP/s",
            "config": {"workload": f"B{B} H{H} L{L} D{D} bf16, lengths U[32,1024], {'causal' if causal else 'non-causal'} + key padding",
                       "computed_pairs_over_valid_pairs": round(pairs / valid_pairs, 3)},
            "ms_per_launch": round(ms, 3),
            "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(tf / peak, 4),
                         "peak_source": peak_kind},
        })
    return out


def run_token_project_sweep(args) -> None:
    """The sequence tokenizer of layer 0 (gather of table rows -> projection 128 -> 512 -> SiLU -> LayerNorm -> position
    rows -> first RMSNorm, residual stream written for the kept rows only) as ONE kernel (`ops.token_project`) against
    the three kernels the engine runs by default (`gather_rows`, `grouped_linear`, `token_tail`)."""
    from taac_2026_b200.inputs import zipf_ids

    peaks, peak_kind = load_peaks()
    rows = args.rows or 1_000_000
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(1_000_001, 128, generator=g, device="cuda").bfloat16()
    ids = zipf_ids(rows, 1_000_000, 1.1, torch.Generator().manual_seed(0)).view(1, rows).cuda()
    w = (torch.randn(512, 128, generator=g, device="cuda") * 128 ** -0.5).bfloat16()
    b = torch.randn(512, generator=g, device="cuda")
    lw, lb, rw = ((1 + 0.02 * torch.randn(512, generator=g, device="cuda")).bfloat16() for _ in range(3))
    pos = torch.randn(1025, 512, generator=g, device="cuda").bfloat16()
    ip = torch.randint(0, 1025, (rows,), generator=g, device="cuda")
    keep = torch.rand(rows, generator=g, device="cuda") < 0.05
    row_dst = torch.where(keep, torch.cumsum(keep, 0) - 1, torch.full_like(ip, -1)).to(torch.int32)
    n_out = int(keep.sum())

    def fused():
        return ops.token_project([table], ids, w, b, lw, lb, pos, ip, None, None, rw, row_dst=row_dst, rows_out=n_out)

    def three():
        x = ops.gather_rows(table, ids[0])
        p = ops.grouped_linear(x, w, b)
        return ops.token_tail(p, lw, lb, pos, ip, None, None, rw, row_dst=row_dst, rows_out=n_out)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    # ids + table rows read, normed rows written, kept rows of the residual stream written
    algo = rows * (8 + 256 + 1024 + 4 + 8) + n_out * 1024
    for name, fn in (("one kernel (token_project)", fused), ("three kernels (gather_rows, grouped_linear, token_tail)", three)):
        for _ in range(3):
            fn()
        times = []
        for _ in range(max(args.steps, 3)):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        ms = statistics.median(times)
        gbs = algo / ms / 1e6
        print(json.dumps({
            "metric": "sequence_tokenizer_rows_per_s", "value": round(rows / ms * 1e3, 1), "unit": "rows/s", "ms": round(ms, 4),
            "config": {"workload": f"{rows} rows, 1 feature x 128 bf16 -> 512, 5 % of the rows kept, {name}", "l2": "256 MB flush between runs"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peak_kind,
                         "note": "bytes of the one-kernel form: ids + table rows in, normed rows and kept residual rows out"},
        }), flush=True)


def run_attention_sweep(args) -> None:
    """Batch 2048 (in slices), 8 heads, head_dim 64, L 1024, lengths uniform in [32, 1024]."""
    peaks, peak_kind = load_peaks()
    batch = args.batch or 256
    if batch <= 512:
        for line in attention_lines(peaks, peak_kind, batch=batch, steps=args.steps, kernel=args.kernel):
            print(json.dumps(line), flush=True)
        return
    # the full configuration (batch 2048) in slices of 256 samples with their own seeds: q, k, v of one slice are
    # 0.8 GB, and the rate of the whole batch is total work over total time
    slices = [attention_lines(peaks, peak_kind, batch=256, steps=args.steps, kernel=args.kernel, seed=i) for i in range((batch + 255) // 256)]
    for which in range(2):
        lines = [sl[which] for sl in slices]
        ms = sum(line["ms_per_launch"] for line in lines)
        work = sum(line["value"] * line["ms_per_launch"] for line in lines)      # TFLOP/s x ms
        tf = work / ms
        merged = dict(lines[0])
        merged["value"] = round(tf, 1)
        merged["ms_per_launch"] = round(ms, 3)
        merged["config"] = {**lines[0]["config"], "workload": lines[0]["config"]["workload"].replace("B256", f"B{256 * len(lines)} ({len(lines)} slices of 256)"),
                            "slice_TFLOPs": [line["value"] for line in lines]}
        merged["roofline"] = {**lines[0]["roofline"], "achieved": round(tf, 1), "frac": round(tf / lines[0]["roofline"]["peak"], 4)}
        print(json.dumps(merged), flush=True)


def run_kept_rows_attention(args) -> None:
    """Packed causal attention in which only the last rows of every sample are queries (`cu_rows_q`): the shape of
    a pyramid block evaluated for the rows it keeps.  Samples of 137..579 rows, 9 + U[0, 16] queries each, 8 heads,
    head_dim 64, bf16 (`--kind kept`); or the first block's own rule (`--kind kept_pyramid`): samples of 137..604
    rows whose queries are 9 rows plus every row beyond the 466th, so that most samples have 9 queries and a fifth
    of them up to 147.  Bound by the stream over K and V."""
    peaks, peak_kind = load_peaks()
    B, H, D = args.batch or 4096, 8, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    if args.kind == "kept_pyramid":
        lens = torch.randint(137, 605, (B,), generator=g, device="cuda")
        keep = 9 + (lens - 466).clamp_min(0)
    else:
        lens = torch.randint(137, 580, (B,), generator=g, device="cuda")
        keep = 9 + torch.randint(0, 17, (B,), generator=g, device="cuda")
    cu = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
    cu[1:] = torch.cumsum(lens, 0)
    cu_q = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
    cu_q[1:] = torch.cumsum(keep, 0)
    rows, q_rows = int(cu[-1]), int(cu_q[-1])
    kv = torch.randn(rows, 2, H, D, generator=g, device="cuda").div_(8).bfloat16()
    q = torch.randn(q_rows, H, D, generator=g, device="cuda").div_(8).bfloat16()
    fn = lambda: ops.varlen_attention(q, kv[:, 0], kv[:, 1], causal=True, cu_rows=cu, max_rows=int(lens.max()),  # noqa: E731
                                      cu_rows_q=cu_q, max_rows_q=int(keep.max()), kernel=args.kernel)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / args.steps
    nbytes = 2.0 * H * D * 2 * (rows + q_rows)
    gbs = nbytes / ms / 1e6
    print(json.dumps({
        "metric": "kept_rows_attention_GBps", "value": round(gbs, 1), "unit": "GB/s",
        "config": {"workload": f"{B} packed samples of {int(lens.min())}..{int(lens.max())} rows, {int(keep.min())}..{int(keep.max())} "
                               f"queries each, H{H} D{D} bf16, causal", "k_rows": rows, "q_rows": q_rows, "kernel": args.kernel},
        "ms_per_launch": round(ms, 3),
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peak_kind},
    }), flush=True)


def run_gather_sweep(args) -> None:
    peaks, peak_kind = load_peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(1_000_001, 128, generator=g, device="cuda").bfloat16()
    from taac_2026_b200.inputs import zipf_ids

    ids = zipf_ids(8192 * 1024, 1_000_000, 1.1, torch.Generator().manual_seed(0)).view(8192, 1, 1024).cuda()
    fn = lambda: ops.sequence_gather([table], ids)  # noqa: E731
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / args.steps
    # Algorithmic HBM bytes: every DISTINCT row is read once (Zipf ids repeat and the repeats are served by
    # the L2), every output row is written, every id is read.
    unique_rows = int(torch.unique(ids).numel())
    nbytes = unique_rows * 256 + ids.numel() * (256 + 8)
    gbs = nbytes / ms / 1e6
    print(json.dumps({
        "metric": "sequence_gather_GBps", "value": round(gbs, 1), "unit": "GB/s",
        "config": {"workload": "8192x1024 Zipf(1.1) ids into a 1000001x128 bf16 table", "distinct_rows": unique_rows},
        "ms_per_launch": round(ms, 3),
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peak_kind},
    }), flush=True)


def measure_fp8_peak() -> float | None:
    """Dense e4m3 GEMM throughput of the library path (torch._scaled_mm, 8192^3), TFLOP/s, best of 5."""
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn).t()
        one = torch.ones((), device="cuda")
        best = None
        for _ in range(6):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
            best = ms if best is None or ms < best else best
        return 2.0 * n**3 / best / 1e9
    except Exception:
        return None


def ffn_lines(peaks: dict, peak_kind: str, *, rows: int, steps: int, fp8_peak: float | None,
              modes=(("gated", False), ("gated", "mx"), ("gated", True), ("plain", False), ("plain", "mx"))) -> list[dict]:
    """`rows` tokens, 512 -> 2 x 2048 (gate, up) -> 512, e4m3 with 1x128 / 128x128 amax scales.  One line per
    (layer kind, precise) pair: the all-e4m3 FFN, and the mode whose up projection runs in bf16 (the one that meets
    5e-2 against the bf16 FFN).  Every line carries its relative error against the bf16 torch FFN on the same data."""
    m, d, hidden = rows, 512, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(m, d, generator=g, device="cuda")
    t4 = torch.randn(m, d, generator=g, device="cuda") / torch.sqrt(torch.randn(m, d, 4, generator=g, device="cuda").pow(2).mean(-1))
    x = torch.where(torch.rand(m, d, generator=g, device="cuda") < 0.01, 3.0 * t4, x).bfloat16()
    del t4
    if fp8_peak is None:
        fp8_peak = measure_fp8_peak()
    out = []
    cache: dict[str, tuple] = {}
    for kind, precise in modes:
        gated = kind == "gated"
        mx = precise == "mx"       # power-of-two scales applied by the block-scaled tensor-core instruction
        if kind not in cache:
            w_up = (torch.randn((2 if gated else 1) * hidden, d, generator=g, device="cuda") * 0.02).bfloat16()
            w_down = (torch.randn(d, hidden, generator=g, device="cuda") * 0.02).bfloat16()
            h = torch.nn.functional.linear(x, w_up)
            h = torch.nn.functional.silu(h[:, :hidden]) * h[:, hidden:] if gated else torch.nn.functional.silu(h)
            ref = torch.nn.functional.linear(h, w_down).float()
            del h
            cache[kind] = (ops.Fp8FfnWeights(w_up, w_down, gated=gated, precise=True), ref,
                           ops.MxFfnWeights(w_up, w_down, gated=gated))
        weights, ref, weights_mx = cache[kind]
        if mx:
            run = lambda: ops.ffn_mx(x, weights_mx)   # noqa: E731
        else:
            run = lambda: ops.ffn_fp8(x, weights, precise=precise)   # noqa: E731
        for _ in range(3):
            got = run()
        torch.cuda.synchronize()
        diff = got.float() - ref
        rel_l2 = (diff.norm() / ref.norm()).item()
        big = ref.abs() > 1e-2
        max_rel = (diff.abs()[big] / ref.abs()[big]).max().item()
        del diff, big, got
        records: list = []
        ops.set_kernel_timing(records)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            run()
        end.record()
        torch.cuda.synchronize()
        ops.set_kernel_timing(None)
        ms = start.elapsed_time(end) / steps
        per = {}
        for name, _meta, s0, s1 in records:
            per[name] = per.get(name, 0.0) + s0.elapsed_time(s1) / steps
        flops = 2.0 * m * d * hidden * (3 if gated else 2)
        tf = flops / ms / 1e9
        tf_gemm = flops / sum(v for k, v in per.items() if "gemm" in k) / 1e9
        nominal = 2.0 * peaks["bf16_tflops"]
        # the precise mode does two thirds (gated) of its FLOPs on the bf16 pipe: its own time floor is not the e4m3 one
        out.append({
            "metric": "ffn_fp8_TFLOPs", "value": round(tf, 1), "unit": "TFLOP/s",
            "config": {"workload": f"{m} tokens, {d} -> {'2x' if gated else ''}{hidden} -> {d}, e4m3 1x128 / 128x128 scales, "
                                   f"{'SiLU-gated' if gated else 'SiLU'}",
                       "mode": ("both projections e4m3, power-of-two scales inside the block-scaled MMA" if mx else
                                "up projection in bf16, down projection e4m3" if precise else "both projections e4m3")},
            "ms_per_step": round(ms, 3), "kernel_ms": {k: round(v, 3) for k, v in per.items()},
            "rel_l2_error_vs_bf16_ffn": round(rel_l2, 5), "max_rel_error_where_ref_above_1e-2": round(max_rel, 3),
            "roofline": {"bound": "tensor", "achieved": round(tf_gemm, 1), "peak": round(fp8_peak, 1) if fp8_peak else nominal,
                         "unit": "TFLOP/s", "frac": round(tf_gemm / (fp8_peak or nominal), 4),
                         "peak_source": "torch._scaled_mm e4m3 8192^3 measured in this run" if fp8_peak else f"2 x bf16 {peak_kind}",
                         "frac_of_2x_bf16_measured": round(tf_gemm / nominal, 4), "note": "achieved = GEMM kernels only; value = whole FFN incl. activation quantisation"},
        })
    return out


def run_ffn_sweep(args) -> None:
    """262 144 tokens, 512 -> 2 x 2048 (gate, up) -> 512, e4m3 with 1x128 / 128x128 amax scales."""
    peaks, peak_kind = load_peaks()
    for line in ffn_lines(peaks, peak_kind, rows=args.rows or 262144, steps=args.steps, fp8_peak=None,
                          modes=(("gated", False), ("gated", "mx"), ("gated", True), ("plain", False), ("plain", "mx"), ("plain", True))):
        print(json.dumps(line), flush=True)


def run_grouped_gemm_sweep(args) -> None:
    """The per-token layers of 9 non-sequence tokens x 8192 samples at d_model 512: this library's grouped GEMM
    with the epilogue inside against the library batched GEMM followed by the separate passes it needs."""
    peaks, peak_kind = load_peaks()
    groups, rows = 9, args.rows or 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    cases = [("qkv projection + bias", 1536, 512, False, False), ("FFN up + bias + SiLU", 2048, 512, True, False),
             ("FFN down + bias + residual", 512, 2048, False, True)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def time_ms(fn) -> float:
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(args.steps):
            flush.zero_()                      # 256 MB > L2: operands start in HBM
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            total += start.elapsed_time(end)
        return total / args.steps

    for name, n, k, silu, with_res in cases:
        x = torch.randn(groups, rows, k, generator=g, device="cuda").bfloat16()
        w = (torch.randn(groups, n, k, generator=g, device="cuda") * k ** -0.5).bfloat16()
        w_t = w.transpose(1, 2).contiguous()
        bias = torch.randn(groups, n, generator=g, device="cuda")
        bias_b = bias.bfloat16().unsqueeze(1)
        res = torch.randn(groups, rows, n, generator=g, device="cuda").bfloat16() if with_res else None
        ours = lambda: ops.grouped_linear(x, w, bias, silu=silu, residual=res)   # noqa: E731
        if with_res:
            lib = lambda: ops.bias_act_rows(torch.baddbmm(res, x, w_t), bias_b, silu=False)   # noqa: E731
        else:
            lib = lambda: ops.bias_act_rows(torch.bmm(x, w_t), bias_b, silu=silu)   # noqa: E731
        ms, ms_lib, ms_bmm = time_ms(ours), time_ms(lib), time_ms(lambda: torch.bmm(x, w_t))
        tf = 2.0 * groups * rows * n * k / ms / 1e9
        print(json.dumps({
            "metric": "grouped_linear_TFLOPs", "value": round(tf, 1), "unit": "TFLOP/s",
            "config": {"workload": f"{groups} groups x {rows} rows, {k} -> {n}, bf16, {name}", "l2": "256 MB flush between launches"},
            "ms_per_launch": round(ms, 4), "library_bmm_plus_epilogue_ms": round(ms_lib, 4), "library_bmm_alone_ms": round(ms_bmm, 4),
            "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": round(tf / peaks["bf16_tflops"], 4), "peak_source": peak_kind},
        }), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=6)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--workload", default="full", choices=[*WORKLOADS, "norm", "attention", "gather", "ffn", "parity"])
    parser.add_argument("--batch", type=int, default=0, help="per-GPU batch override")
    parser.add_argument("--micro-batch", type=int, default=0)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--launch-log", default="", help="write every recorded launch of the timing pass (name, ms, shape) to this file")
    parser.add_argument("--profile", action="store_true",
                        help="run --warmup untimed and --steps plain steps of the main workload and exit (for ncu)")
    parser.add_argument("--ffn", choices=["fp8", "fp8_mx", "fp8_precise", "bf16"], default="fp8", help="shared FFN of every block")
    parser.add_argument("--host-format", choices=["compact32", "padded64"], default="compact32",
                        help="what the end-to-end arm copies per step: the compact 32-bit sequence record "
                             "(inputs.compact_model_input, expanded on the device) or the reference's padded int64 record")
    parser.add_argument("--padded", action="store_true", help="reference [B, T, d] layout instead of packed valid tokens")
    parser.add_argument("--late-select", action="store_true",
                        help="apply the pyramid's row selection after the whole block (the reference's order) instead of "
                             "right after attention")
    parser.add_argument("--rotate", type=int, default=4, help="distinct batches per rank that rotate through the timed steps")
    parser.add_argument("--min-timed-s", type=float, default=2.0, help="repeat the K-step pass until an arm has run about this long")
    parser.add_argument("--parity-rows", type=int, default=256,
                        help="rows scored by both the GPU and the CPU arm after the timed regions (scores, AUC)")
    parser.add_argument("--no-op-lines", action="store_true", help="skip the standalone attention / FFN lines of the default run")
    parser.add_argument("--no-reference-order", action="store_true", help="skip the pass in the reference's order of operations")
    parser.add_argument("--fused-tokenizer", action="store_true",
                        help="sequence tokenizer as the one-kernel form (ops.token_project) instead of gather, projection and tail kernels")
    parser.add_argument("--no-prepare-ahead", action="store_true",
                        help="end-to-end arm: run duplicate removal and the row plan inside the forward (one device drain per "
                             "batch) instead of on the copy stream under the previous batch")
    parser.add_argument("--rows", type=int, default=0)
    parser.add_argument("--cols", type=int, default=0)
    parser.add_argument("--kind", default="")
    parser.add_argument("--kernel", type=int, default=0)
    args = parser.parse_args()
    if args.workload == "norm":
        if args.kind == "token_tail":
            run_token_tail_sweep(args)
        elif args.kind == "bwd":
            run_norm_backward_sweep(args)
        elif args.kind == "token_project":
            run_token_project_sweep(args)
        else:
            run_norm_sweep(args)
    elif args.workload == "attention":
        if args.kind in ("kept", "kept_pyramid"):
            run_kept_rows_attention(args)
        else:
            run_attention_sweep(args)
    elif args.workload == "gather":
        run_gather_sweep(args)
    elif args.workload == "ffn":
        if args.kind == "grouped":
            run_grouped_gemm_sweep(args)
        else:
            run_ffn_sweep(args)
    elif args.workload == "parity":
        run_parity_stages(args)
    else:
        run_e2e(args)


if __name__ == "__main__":
    main()
