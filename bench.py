"""Benchmark of the MD hot path: atom-steps/s of Langevin NVT steps (neighbour check + compaction + energy, forces and
stress + both half kicks) of the random-initialised MACE "medium" model on 1,944-atom NaCl.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line. ``value`` is the throughput of captured whole-step graphs with the noise already resident on
the device (timed with CUDA events on the replay stream); ``e2e`` is the same metric through the public API
(``B200Engine.step``) with the noise drawn on the host and uploaded from pinned memory and a device-to-host read of
the step's energy inside the timed region. ``roofline`` describes the stage with the largest share of the force call,
timed with CUDA events in an eager pass: ``achieved`` divides the stage's COMPULSORY bytes (every operand moved once,
the per-edge radial weights never leaving the chip) by its time, ``design_bytes`` is what the kernels as built move,
``traffic`` the DRAM bytes ncu measured. ``cpu_baseline`` times whole MD steps of the CPU oracle (NumPy Langevin, the
oracle's neighbour list, the fp32 PyTorch model on all host cores) on the SAME configuration, a few steps of it.
``--impl reference`` times that CPU path alone (the third-party model the reference calls is not installable here,
so the CPU arm is the oracle port).

With N > 1 (launched under torch.distributed.run) the default workload is the spatially decomposed 884,736-atom cell
(strong scaling: the line carries its own single-GPU time of the same cell); a workload named with --workload that is
not decomposed runs as independent replicas.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

WORKLOADS = {
    # name: (model, structure builder args, temperature, avg_num_neighbors)
    "medium_nacl_1944_langevin": dict(model="medium", seed=1, repeat=(9, 9, 3), sigma=0.05, temperature=300.0),
    "small_nacl_216_langevin": dict(model="small", seed=0, repeat=(3, 3, 3), sigma=0.05, temperature=300.0),
    # 13,824-site random 5-species FCC alloy (primitive cell 24^3), large model, 1,000 K
    "large_alloy_13824_langevin": dict(model="large", seed=2, builder="fcc_alloy", repeat=(24, 24, 24), sigma=0.1,
                                       temperature=1000.0, avg_num_neighbors=54.0),
    # 110,592-atom amorphous Si-O box at 2.2 g/cm^3 (about 59 neighbours per atom at 6 A), medium model
    "medium_sio2_110592_langevin": dict(model="medium", seed=1, builder="silica", temperature=300.0,
                                        avg_num_neighbors=60.0),
}
DEFAULT_WORKLOAD = "medium_nacl_1944_langevin"
# the spatially decomposed configuration (884,736-atom NaCl, 48 x 48 x 48 cells): the default at --gpus > 1
DOMAIN_WORKLOAD = "medium_nacl_884736_langevin"
DOMAIN_WORKLOADS = {
    DOMAIN_WORKLOAD: dict(model="medium", seed=1, repeat=(48, 48, 48), sigma=0.05, temperature=300.0, max_steps=200),
    "medium_nacl_110592_langevin": dict(model="medium", seed=1, repeat=(24, 24, 24), sigma=0.05, temperature=300.0,
                                        max_steps=200),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            p = json.load(handle)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            try:
                sm.append(float(row[1]))
                sm_max = float(row[2])
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, row[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=sm_max, reasons=sorted(reasons),
                    samples=len(sm))


def build_problem(workload: str, device):
    import dataclasses

    from fastmace_b200.engine import B200Engine
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.model import SPECS, init_weights
    from fastmace_b200.state import SimulationState
    from fastmace_b200.structures import fcc_alloy, nacl, silica

    w = WORKLOADS[workload]
    spec = dataclasses.replace(SPECS[w["model"]], avg_num_neighbors=w.get("avg_num_neighbors", 32.0))
    weights = init_weights(spec, w["seed"])
    builder = w.get("builder", "nacl")
    if builder == "nacl":
        structure = nacl(w["repeat"], w["sigma"], w["seed"])
    elif builder == "fcc_alloy":
        structure = fcc_alloy(w["repeat"], w["sigma"], w["seed"])
    else:
        structure = silica(seed=w["seed"])
    structure = structure.with_velocities(w["temperature"], w["seed"] + 100)
    ff = B200ForceField(spec, weights, structure.numbers, structure.cell, compute_stress=True, device=device)
    state = SimulationState.from_structure(structure, ff.device, seed=w["seed"], compute_stress=True)
    integrator = Langevin(state, IntegratorConfig(timestep_fs=1.0), temperature_K=w["temperature"])
    engine = B200Engine(ff, integrator, state, mode="graph", check_every=0)
    return spec, weights, structure, ff, state, integrator, engine


def compulsory_bytes(spec, n_atoms: int, n_edges: int, n_species: int = 2) -> dict:
    """Bytes per force call each timed stage cannot avoid: node rows read or written once, per edge its index, vector,
    harmonics and the 64 hidden radial features -- the per-edge tensor-product weights [P * C] are a product of those
    64 features and are counted as never leaving the chip. ``roofline.achieved`` follows these."""
    c = spec.channels
    hid = (spec.hidden_lmax + 1) ** 2
    from fastmace_b200 import so3
    m1 = so3.mid_dim(spec.paths(1))
    out = {}
    out["edge_features"] = n_edges * (8 + 12) + n_atoms * 24 + n_edges * (16 + 64 + 2 * 2 * 64 * 4)
    out["radial_gemm"] = n_edges * 2 * 64 * 4                 # reads the hidden features; its output is on-chip in the target design
    out["tp_forward_l0"] = n_edges * (64 * 4 + 64 + 4) + n_atoms * 16 * n_species * 64 * 4
    out["tp_forward_l1"] = n_edges * (64 * 4 + 64 + 4) + n_atoms * (m1 + hid) * c * 4
    out["tp_backward_l0"] = n_edges * (2 * 64 * 4 + 64 + 16 + 4 + 16) + n_atoms * (16 * n_species * 64 * 4 + 36)
    out["tp_backward_l1"] = n_edges * (2 * 64 * 4 + 64 + 16 + 4 + 16) + n_atoms * ((m1 + 2 * hid) * c * 4 + 36)
    return out


def design_bytes(spec, n_atoms: int, n_edges: int, n_species: int = 2) -> dict:
    """Bytes the kernels as built move per force call: the compulsory ones plus the per-edge radial weights in HBM
    (values and d/dr, 4 P C bytes each, written once and read by the tensor-product kernels) and the per-edge
    hand-over of the sender gradient (written by the adjoint, read back by the gather)."""
    c = spec.channels
    hid = (spec.hidden_lmax + 1) ** 2
    p1 = len(spec.paths(1))
    out = dict(compulsory_bytes(spec, n_atoms, n_edges, n_species))
    out["radial_gemm"] += n_edges * 2 * p1 * c * 4
    out["tp_forward_l1"] += n_edges * p1 * c * 4
    out["tp_backward_l0"] += n_edges * 16 * 64 * 4
    out["tp_backward_l1"] += n_edges * (2 * p1 * c * 4 + 2 * hid * c * 4)
    return out


def measured_traffic(stage: str, n_edges: int):
    """DRAM bytes (read + write) of the stage's launches for ``n_edges`` edges, scaled per edge from the ncu capture
    recorded in ``profiles/`` (lines ``stage <name> edges <E> dram_bytes <B>``); None when no capture is recorded."""
    import glob
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "ncu_dram_bytes_*.txt"))):
        with open(path) as handle:
            for line in handle:
                words = line.split()
                if len(words) >= 6 and words[0] == "stage" and words[1] == stage:
                    return float(words[5]) / float(words[3]) * n_edges
    return None


class CpuReferenceMD:
    """Whole MD steps of the CPU oracle on a workload's own configuration: NumPy Langevin half steps, displacement
    test, rebuild when it fires, compaction, the fp32 PyTorch model on every host core, second half kick -- the
    checked step of the reference (``fastmace/engine/graph.py:968-998``) with the oracle in place of the
    third-party model."""

    def __init__(self, workload: str):
        import dataclasses

        from fastmace_b200.model import SPECS, init_weights
        from fastmace_b200.structures import FS, KB, fcc_alloy, nacl, silica
        from oracle import mace_oracle, neighbours_oracle
        from oracle.langevin_oracle import LangevinOracle

        w = {**WORKLOADS, **DOMAIN_WORKLOADS}[workload]
        self.mace, self.nl = mace_oracle, neighbours_oracle
        self.spec = dataclasses.replace(SPECS[w["model"]], avg_num_neighbors=w.get("avg_num_neighbors", 32.0))
        self.weights = init_weights(self.spec, w["seed"])
        builder = w.get("builder", "nacl")
        s = nacl(w["repeat"], w["sigma"], w["seed"]) if builder == "nacl" else \
            fcc_alloy(w["repeat"], w["sigma"], w["seed"]) if builder == "fcc_alloy" else silica(seed=w["seed"])
        s = s.with_velocities(w["temperature"], w["seed"] + 100)
        self.structure = s
        self.skin = 0.3
        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        self.x, self.v = s.positions.copy(), s.velocities.copy()
        self.langevin = LangevinOracle(s.masses, 1.0 * FS, 0.01 / FS, w["temperature"], KB)
        self.rng = np.random.default_rng(w["seed"])
        self.rebuilds = 0
        self._rebuild()
        self.energy, self.f = self._forces()

    def _rebuild(self):
        self.candidates = self.nl.build_screened(self.x, self.structure.cell, self.spec.r_cut, self.skin)
        self.reference_positions = self.x.copy()
        self.rebuilds += 1

    def _forces(self):
        s = self.structure
        snd, rcv, unit, _, count = self.nl.compact(self.x, s.cell, *self.candidates, self.spec.r_cut)
        e, f, _ = self.mace.evaluate(self.spec, self.weights, self.x, s.cell, s.numbers, snd[:count], rcv[:count],
                                     unit[:count], dtype=torch.float32)
        return float(e), f.numpy().astype(np.float64)

    def step(self):
        noise = self.rng.standard_normal((2, self.structure.natoms, 3))
        self.x, self.v = self.langevin.first_half(self.x, self.v, self.f, noise[0], noise[1])
        if self.nl.needs_rebuild(self.x, self.reference_positions, self.skin):
            self._rebuild()
        self.energy, self.f = self._forces()
        self.v = self.langevin.second_half(self.v, self.f)

    def time_steps(self, steps: int, warmup: int, budget_s: float):
        """Times up to ``steps`` steps after ``warmup`` untimed ones, stopping early once ``budget_s`` seconds of
        timed work are done (at least two steps). Returns (seconds per step, steps timed)."""
        for _ in range(warmup):
            self.step()
        done, t0 = 0, time.perf_counter()
        while done < steps:
            self.step()
            done += 1
            if done >= 2 and time.perf_counter() - t0 > budget_s:
                break
        return (time.perf_counter() - t0) / done, done


def cpu_baseline_block(workload: str, steps: int, warmup: int, budget_s: float):
    md = CpuReferenceMD(workload)
    seconds, done = md.time_steps(steps, warmup, budget_s)
    n = md.structure.natoms
    return dict(value=n / seconds, unit="atom-steps/s", cores=md.threads, kind="port",
                sample=f"{done} whole MD steps (after {warmup} untimed) of the CPU oracle on the workload itself "
                       f"({n} atoms, fp32 model on {md.threads} threads, {seconds:.2f} s per step)",
                ms_per_step=1e3 * seconds, steps=done), md


def run_reference(args):
    """The CPU arm: the oracle port of the reference's checked step on this workload's configuration. The third-party
    model the reference evaluates (mace-torch) is not installable here. Steps beyond a time budget are not run and
    ``steps`` reports how many were timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # a step of a decomposed workload (10^5 - 10^6 atoms) takes many minutes on the host: its sample is the
    # 1,944-atom cell of the same crystal, model and thermostat (the cost per atom does not depend on the cell size)
    workload = args.workload if args.workload in WORKLOADS else DEFAULT_WORKLOAD
    warmup = max(1, min(args.warmup, 2))
    block, md = cpu_baseline_block(workload, args.steps, warmup, budget_s=120.0)
    if workload != args.workload:
        block["sample"] += f"; stands in for {args.workload} (same crystal, model and thermostat)"
    line = dict(metric="md_atom_steps_per_s", value=block["value"], unit="atom-steps/s", n_gpus=args.gpus,
                steps=block["steps"], warmup=warmup, requested_steps=args.steps, requested_warmup=args.warmup,
                ms_per_step=block["ms_per_step"], us_per_step=1e3 * block["ms_per_step"], higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(workload=args.workload, sampled_workload=workload, atoms=md.structure.natoms,
                            model={**WORKLOADS}[workload]["model"],
                            integrator="langevin_nvt_1fs_0.01perfs", neighbour_rebuilds=md.rebuilds,
                            note="CPU oracle port of the reference's checked MD step; the third-party model the "
                                 "reference evaluates (mace-torch) cannot be installed here"),
                cpu_baseline={k: block[k] for k in ("value", "unit", "cores", "kind", "sample")},
                e2e=dict(value=block["value"], unit="atom-steps/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def time_single_gpu_cell(w, spec, weights, structure, device, steps: int, warmup: int):
    """ms per step of the decomposed workload's cell on ONE GPU through the plain periodic force field and the checked
    engine (no bricks, no halo atoms, counter-based noise like the ranks): the denominator of the strong-scaling
    efficiency. Returns (ms per step, description); everything it allocated is released before it returns."""
    from fastmace_b200.engine import B200Engine
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.state import SimulationState
    ff = B200ForceField(spec, weights, structure.numbers, structure.cell, compute_stress=True, device=device)
    state = SimulationState.from_structure(structure, ff.device, seed=w["seed"], compute_stress=True)
    integrator = Langevin(state, IntegratorConfig(timestep_fs=1.0), temperature_K=w["temperature"], noise="device",
                          device_seed=w["seed"])
    engine = B200Engine(ff, integrator, state, mode="checked")
    for _ in range(warmup):
        engine.step()
    engine.flush()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        engine.step()
    stop.record()
    stop.synchronize()
    ms = start.elapsed_time(stop) / steps
    note = (f"{steps} steps after {warmup}: plain periodic force field, checked engine, "
            f"{'per-edge hand-over' if ff.edge_local else 'mirror-evaluation'} adjoint, "
            f"{int(ff.edge_count.item())} edges")
    del engine, integrator, state, ff
    torch.cuda.empty_cache()
    return ms, note


def run_domain(args, world, rank, local_rank, device):
    """The spatially decomposed configuration: one brick per rank, partitioned MD state, four halo exchanges and three
    small all-reduces per step (``fastmace_b200.halo.DomainSimulation``), timed through its public ``step``. With one
    rank the same cell runs through the plain single-GPU engine."""
    import dataclasses

    import torch.distributed as dist

    from fastmace_b200 import _lib
    from fastmace_b200.halo import DistributedTransport, DomainSimulation
    from fastmace_b200.model import SPECS, init_weights
    from fastmace_b200.structures import nacl

    w = DOMAIN_WORKLOADS[args.workload]
    lib = _lib.load()
    spec = dataclasses.replace(SPECS[w["model"]], avg_num_neighbors=32.0)
    weights = init_weights(spec, w["seed"])
    structure = nacl(w["repeat"], w["sigma"], w["seed"]).with_velocities(w["temperature"], w["seed"] + 100)
    n_atoms = structure.natoms
    steps = min(args.steps, w["max_steps"])
    warmup = min(max(3, args.warmup), 10)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(ms):
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    pk = peaks()
    common = dict(metric="md_atom_steps_per_s", unit="atom-steps/s", n_gpus=world, steps=steps, warmup=warmup,
                  higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic")
    if world == 1:
        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = lib.fmb_launch_count()
        ms, note = time_single_gpu_cell(w, spec, weights, structure, device, steps, warmup)
        launches = int(lib.fmb_launch_count() - launches0)
        line = dict(common, value=n_atoms / (ms * 1e-3), ms_per_step=ms, us_per_step=1e3 * ms,
                    config=dict(workload=args.workload, atoms=n_atoms, model=w["model"],
                                integrator="langevin_nvt_1fs_0.01perfs_device_noise", parallelism="1gpu", note=note,
                                l2="per-step working set far exceeds the 126 MB L2; no flush"),
                    clocks=sampler.stop(),
                    e2e=dict(value=n_atoms / (ms * 1e-3), unit="atom-steps/s", h2d_bytes_per_step=0,
                             d2h_bytes_per_step=4, ms_per_step=ms,
                             note="state and noise live on the device; per step the host reads the rebuild flag"),
                    gpu_launches=launches, launches_per_step=launches / (steps + warmup))
        print(json.dumps(line))
        return

    # the same cell on one GPU, measured on rank 0 before the ranks start (the others wait at the barrier)
    single_ms, single_note = None, None
    if rank == 0 and not args.no_single_gpu_baseline:
        single_ms, single_note = time_single_gpu_cell(w, spec, weights, structure, device, 5, 2)
    barrier()
    sim = DomainSimulation(spec, weights, structure, world, temperature_K=w["temperature"], seed=w["seed"],
                           device=device, ranks=[rank], transport=DistributedTransport())
    initial_energy = sim.potential_energy()
    for _ in range(warmup):
        sim.step()
    sim.flush()
    launches0 = lib.fmb_launch_count()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        sim.step()
    stop.record()
    stop.synchronize()
    barrier()
    clocks = sampler.stop()
    total_ms = reduce_max(start.elapsed_time(stop))
    launches = int(lib.fmb_launch_count() - launches0)
    sim.flush()
    # end to end: further steps of the same run with the step's energy read back to the host every step
    e2e_steps = min(steps, 50)
    pinned = torch.zeros(e2e_steps, dtype=torch.float64).pin_memory()
    barrier()
    t0 = time.perf_counter()
    for k in range(e2e_steps):
        sim.step()
        pinned[k:k + 1].copy_(sim.energy, non_blocking=True)
    sim.flush()
    barrier()
    e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3)
    assert bool(torch.isfinite(pinned).all()), "non-finite energies"
    # stage timing of this rank's three phases (no exchange in between: the halo rows keep the last step's values)
    r = sim.ranks[0]
    lib.fmb_profile_enable(1)
    for k in range(3):
        if k == 1:
            _lib.profile_read()
        for phase in range(3):
            r.ff.phase(phase, r.x_local)
    stages = _lib.profile_read()
    lib.fmb_profile_enable(0)
    stage_ms = {k: v[0] / 2 for k, v in stages.items()}
    info = sim.info()
    n_edges = info["local_edges"]
    algo = compulsory_bytes(spec, info["local_atoms"], n_edges)
    top = max((k for k in stage_ms if k in algo), key=lambda k: stage_ms[k])
    achieved = algo[top] / (stage_ms[top] * 1e-3) / 1e9
    owned, local = info["owned_all"], info["local_all"]
    counts = torch.tensor([float(owned[0]), float(local[0]), float(len(r.part.send_index))], device=device,
                          dtype=torch.float64)
    gathered = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(gathered, counts)
    owned_all = [int(g[0]) for g in gathered]
    local_all = [int(g[1]) for g in gathered]
    sent_all = [int(g[2]) for g in gathered]
    hid = (spec.hidden_lmax + 1) ** 2
    row = hid * spec.channels * 4
    strong = None
    if single_ms is not None:
        strong = dict(single_gpu_ms_per_step=single_ms, ms_per_step=total_ms / steps,
                      speedup=single_ms / (total_ms / steps), efficiency=single_ms / (world * total_ms / steps),
                      single_gpu=single_note)
    line = dict(common, value=n_atoms * steps / (total_ms * 1e-3), ms_per_step=total_ms / steps,
                us_per_step=1e3 * total_ms / steps,
                config=dict(workload=args.workload, atoms=n_atoms, model=w["model"],
                            integrator="langevin_nvt_1fs_0.01perfs_device_noise",
                            parallelism=f"bricks{'x'.join(map(str, info['bricks']))}_halo_exchange",
                            owned_atoms=owned_all, local_atoms=local_all,
                            local_over_owned=max(l / max(1, o) for l, o in zip(local_all, owned_all)),
                            halo_rows_sent=sent_all, local_edges_rank0=n_edges, initial_energy_eV=initial_energy,
                            repartitions=info["repartitions"], repartition_seconds=info["repartition_seconds"],
                            repartition_seconds_each=info["repartition_log"],
                            exchanges="per step: positions (24 B), x rows and their gradient (%d B each), forces (12 B) per "
                                      "halo atom over NCCL all_to_all; all-reduces of 10 + 10 float64 and one flag" % row,
                            nvlink_bytes_per_step_rank0=sent_all[0] * (24 + 2 * row + 12),
                            l2="per-step working set far exceeds the 126 MB L2; no flush"),
                clocks=clocks, strong_scaling=strong,
                e2e=dict(value=n_atoms * e2e_steps / (e2e_ms * 1e-3), unit="atom-steps/s", h2d_bytes_per_step=0,
                         d2h_bytes_per_step=8 + 4, ms_per_step=e2e_ms / e2e_steps, steps=e2e_steps,
                         note="state and noise live on the device; per step the host reads the rebuild flag and the energy"),
                gpu_launches=launches, launches_per_step=launches / steps,
                roofline=dict(bound="hbm", kernel=top, achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s",
                              frac=achieved / pk["hbm_gbs"], traffic=None, peak_source=pk["source"],
                              algorithmic_bytes=algo[top], stage_ms={k: round(v, 4) for k, v in stage_ms.items()},
                              note="rank 0's three phases, compulsory bytes of its local atoms and edges"))
    if rank == 0:
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=1000)
    parser.add_argument("--warmup", type=int, default=100)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + sorted(DOMAIN_WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-single-gpu-baseline", action="store_true",
                        help="decomposed workloads: skip timing the same cell on one GPU (the strong_scaling block)")
    args = parser.parse_args()
    if args.workload is None:
        args.workload = DOMAIN_WORKLOAD if int(os.environ.get("WORLD_SIZE", "1")) > 1 else DEFAULT_WORKLOAD
    if args.impl == "reference":
        run_reference(args)
        return

    from fastmace_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise _lib.Fmb200Error("bench.py needs a CUDA device (there is no CPU path for the product)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()
    if args.workload in DOMAIN_WORKLOADS:
        run_domain(args, world, rank, local_rank, device)
        return

    spec, weights, structure, ff, state, integrator, engine = build_problem(args.workload, device)
    n_atoms = structure.natoms
    warmup = max(3, args.warmup)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-resident throughput (value)
    launches_before = lib.fmb_launch_count()
    engine.run(1)                      # captures the step graph
    launches_per_step = None
    for _ in range(warmup - 1):
        engine.step()
    engine.flush()
    # both timed loops integrate the same stretch of the trajectory: the random-init model pulls the crystal together
    # over a few hundred steps (the edge count grows by ~20 %), so the state is put back before the end-to-end loop
    saved = {name: getattr(state, name).clone() for name in ("positions", "velocities", "forces", "energy")}
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms, done = 0.0, 0
    while done < args.steps:
        # refill the drawn-ahead noise outside the timed region: `value` has its inputs resident in HBM
        integrator.refill(state)
        todo = min(integrator.rows, args.steps - done)
        torch.cuda.synchronize()
        start.record()
        for _ in range(todo):
            engine.graph.replay()
        stop.record()
        stop.synchronize()
        total_ms += start.elapsed_time(stop)
        state.rng.cursor = integrator.rows          # used up as far as the host is concerned
        done += todo
    clocks = sampler.stop()
    engine.flush()
    if world > 1:
        t = torch.tensor([total_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * n_atoms * args.steps / (total_ms * 1e-3)

    # ---------------------------------------------------------------- end to end through the public API (e2e)
    # a run as a user starts it: a fresh integrator, engine and noise stream on the same force field, stepping the
    # same stretch of the trajectory through B200Engine.step() (host noise drawn and uploaded from pinned memory as
    # the steps consume it, the step's energy read back every step)
    from fastmace_b200.engine import B200Engine
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.state import RandomStream
    pinned = torch.zeros(args.steps, dtype=torch.float64).pin_memory()
    for name, value_ in saved.items():
        getattr(state, name).copy_(value_)
    state.rng = RandomStream(np.random.default_rng(WORKLOADS[args.workload]["seed"] + 1))
    user_integrator = Langevin(state, IntegratorConfig(timestep_fs=1.0), temperature_K=WORKLOADS[args.workload]["temperature"])
    user_engine = B200Engine(ff, user_integrator, state, mode="graph")      # the defaults, check points included
    user_engine.step()                 # untimed: captures the step graph (warm-ups restore the state)
    user_engine.flush()
    barrier()
    t0 = time.perf_counter()
    start.record()
    for k in range(args.steps):
        user_engine.step()                              # host noise draw + upload when the batch runs out
        pinned[k:k + 1].copy_(state.energy, non_blocking=True)
    stop.record()
    stop.synchronize()
    e2e_ms = start.elapsed_time(stop)
    user_engine.flush()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max(e2e_ms, wall_ms)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * n_atoms * args.steps / (e2e_ms * 1e-3)
    assert bool(torch.isfinite(pinned).all()), "non-finite energies in the end-to-end run"
    engine = user_engine

    # ---------------------------------------------------------------- launches per step and per-stage timing
    before = lib.fmb_launch_count()
    engine._device_step()
    torch.cuda.synchronize()
    launches_per_step = int(lib.fmb_launch_count() - before)
    n_edges = int(ff.edge_count.item())
    lib.fmb_profile_enable(1)
    profile_calls = 20
    for _ in range(3):
        ff(state.positions)
    _lib.profile_read()
    for _ in range(profile_calls):
        ff(state.positions)
    stages = _lib.profile_read()
    lib.fmb_profile_enable(0)
    stage_ms = {k: v[0] / profile_calls for k, v in stages.items()}
    force_ms = sum(stage_ms.values())
    n_species = len(set(int(z) for z in structure.numbers))
    algo = compulsory_bytes(spec, n_atoms, n_edges, n_species)
    design = design_bytes(spec, n_atoms, n_edges, n_species)
    top = max((k for k in stage_ms if k in algo), key=lambda k: stage_ms[k])
    pk = peaks()
    achieved = algo[top] / (stage_ms[top] * 1e-3) / 1e9
    traffic = measured_traffic(top, n_edges) if args.workload == DEFAULT_WORKLOAD else None
    roofline = dict(bound="hbm", kernel=top, achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s",
                    frac=achieved / pk["hbm_gbs"], traffic=traffic, peak_source=pk["source"],
                    ms_per_launch=stage_ms[top] / max(1, stages[top][1] // profile_calls),
                    algorithmic_bytes=algo[top], design_bytes=design[top],
                    design_frac=design[top] / (stage_ms[top] * 1e-3) / 1e9 / pk["hbm_gbs"],
                    share_of_force_call=stage_ms[top] / force_ms,
                    stage_ms={k: round(v, 5) for k, v in stage_ms.items()},
                    stage_frac={k: round(algo[k] / (stage_ms[k] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                                for k in stage_ms if k in algo and stage_ms[k] > 0})

    line = dict(metric="md_atom_steps_per_s", value=value, unit="atom-steps/s", n_gpus=world, steps=args.steps,
                warmup=warmup, ms_per_step=ms_per_step, us_per_step=1e3 * ms_per_step, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload, atoms=n_atoms, edges=n_edges, model=WORKLOADS[args.workload]["model"],
                            integrator="langevin_nvt_1fs_0.01perfs", parallelism=f"replicas{world}" if world > 1 else "1gpu",
                            l2="per-step working set (radial weight tensors, > 600 MB) exceeds the 126 MB L2; no flush",
                            neighbour_rebuilds=ff.neighbours.rebuilds),
                clocks=clocks,
                e2e=dict(value=e2e_value, unit="atom-steps/s", h2d_bytes_per_step=2 * n_atoms * 3 * 8,
                         d2h_bytes_per_step=8, ms_per_step=e2e_ms / args.steps),
                gpu_launches=launches_per_step * args.steps, launches_per_step=launches_per_step,
                roofline=roofline)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        block, _ = cpu_baseline_block(args.workload, 2, 1, budget_s=30.0)
        line["cpu_baseline"] = {k: block[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
