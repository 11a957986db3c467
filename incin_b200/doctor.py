"""Environment report, plan report and tuning report (crates/incin/src/doctor.rs:55-82, plan_report.rs:10-97,
tune_report.rs:7-94).  ``Host`` is the probe interface so the reports can be tested against a fake machine."""
from __future__ import annotations

import json
import os
import platform
import shutil
from dataclasses import asdict, dataclass, field
from typing import Protocol

from .core.device import DeviceKind
from .core.spec import REGISTRIES


class Host(Protocol):
    def python(self) -> str: ...
    def torch_version(self) -> str: ...
    def cuda_devices(self) -> list[dict]: ...
    def tools(self) -> dict[str, str | None]: ...
    def libraries(self) -> dict[str, bool]: ...


class RealHost:
    def python(self) -> str:
        return platform.python_version()

    def torch_version(self) -> str:
        import torch
        return torch.__version__

    def cuda_devices(self) -> list[dict]:
        import torch
        out = []
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                out.append({"index": i, "name": p.name, "arch": f"sm_{p.major}{p.minor}", "sms": p.multi_processor_count,
                            "memory_gib": round(p.total_memory / 2 ** 30, 1),
                            "peers": [j for j in range(torch.cuda.device_count())
                                      if j != i and torch.cuda.can_device_access_peer(i, j)]})
        return out

    def tools(self) -> dict[str, str | None]:
        return {t: shutil.which(t) for t in ("nvcc", "g++", "ncu", "nvidia-smi")}

    def libraries(self) -> dict[str, bool]:
        from . import _native
        return {"libincin_sm100.so": _native.cuda_library_path().exists(),
                "libincin_host.so": _native.host_library_path().exists()}


@dataclass
class Finding:
    level: str       # ok | warn | error
    code: str
    detail: str


@dataclass
class DoctorReport:
    python: str
    torch: str
    devices: list
    tools: dict
    libraries: dict
    findings: list = field(default_factory=list)

    @property
    def healthy(self) -> bool:
        return not any(f.level == "error" for f in self.findings)

    def to_json(self) -> str:
        d = asdict(self)
        d["healthy"] = self.healthy
        return json.dumps(d, indent=1)

    def to_text(self) -> str:
        lines = [f"python {self.python}, torch {self.torch}"]
        for d in self.devices:
            lines.append(f"  cuda:{d['index']} {d['name']} {d['arch']} {d['sms']} SMs {d['memory_gib']} GiB peers={d['peers']}")
        if not self.devices:
            lines.append("  no CUDA device visible: the CPU backend (the default) is the only backend")
        lines += [f"  {k}: {v or 'missing'}" for k, v in self.tools.items()]
        lines += [f"  {k}: {'built' if v else 'not built (python -m incin_b200 build)'}" for k, v in self.libraries.items()]
        lines += [f"[{f.level}] {f.code}: {f.detail}" for f in self.findings]
        return "\n".join(lines)


def doctor(host: Host | None = None) -> DoctorReport:
    host = host or RealHost()
    rep = DoctorReport(host.python(), host.torch_version(), host.cuda_devices(), host.tools(), host.libraries())
    for d in rep.devices:
        if d["arch"] != "sm_100":
            rep.findings.append(Finding("error", "arch-unsupported",
                                        f"cuda:{d['index']} is {d['arch']}; the kernels are built for sm_100a only"))
    if rep.devices and not rep.libraries.get("libincin_sm100.so"):
        rep.findings.append(Finding("error", "native-missing", "a GPU is present but libincin_sm100.so is not built"))
    if not rep.libraries.get("libincin_host.so"):
        rep.findings.append(Finding("warn", "host-missing", "libincin_host.so is not built: CPU oracle and rendezvous unavailable"))
    if rep.tools.get("nvcc") is None:
        rep.findings.append(Finding("warn", "nvcc-missing", "nvcc not found: the CUDA library cannot be rebuilt here"))
    if len(rep.devices) > 1:
        lonely = [d["index"] for d in rep.devices if len(d["peers"]) < len(rep.devices) - 1]
        if lonely:
            rep.findings.append(Finding("warn", "peer-access", f"GPUs {lonely} cannot map every peer: fused collectives need NVLink/P2P"))
    if not rep.findings:
        rep.findings.append(Finding("ok", "all-good", "every probe passed"))
    return rep


def capability_report() -> str:
    from .core.spec import capability_table_markdown
    return capability_table_markdown()


def plan_report(world: int, *, params: int, layers: int, hidden: int, batch: int, seq: int, shard_extent: int,
                objective: str = "step_time") -> str:
    """Candidate (dp, tp, pp) meshes with the planner's memory / communication / time estimates."""
    from .parallel.planner import HybridPlanner, HybridWorkload, PlanObjective
    wl = HybridWorkload(batch, seq, params, layers, hidden, 6.0 * params, shard_extent, microbatches=max(1, batch // 4))
    pl = HybridPlanner(world)
    lines = [f"world={world} params={params / 1e9:.2f}B batch={batch}x{seq}"]
    for m in pl.candidates():
        lines.append("  " + pl.estimate(m, wl).explain())
    try:
        best = pl.plan(wl, PlanObjective(objective))
        lines.append(f"chosen ({objective}): dp={best.mesh.dp} tp={best.mesh.tp} pp={best.mesh.pp}")
    except ValueError as e:
        lines.append(str(e))
    return "\n".join(lines)


def tune_report() -> str:
    from .tuning import PersistentCache, service
    svc = service()
    recs = PersistentCache().load()
    lines = [f"policy={svc.policy.value} identity={svc.identity.token()} cache={PersistentCache().path} records={len(recs)}"]
    for k, r in list(recs.items())[-40:]:
        lines.append(f"  {r.key}: {r.best} {r.best_ms:.4f} ms ({r.source})")
    return "\n".join(lines)
