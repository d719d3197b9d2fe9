"""SLURM launcher: ``python -m lingua_b200.stool script=apps.main.train config=<yaml> nodes=N ...``

Prepares a dump directory (copy of the ``*.py`` tree, ``base_config.yaml``, ``submit.slurm``) and
submits it, as lingua/stool.py does (StoolArgs :16, SBATCH template :39 with the pre-emption
signal ``USR2@120`` the train loop listens for, launch_job :152). ``launcher=bash`` runs the
script inside an existing allocation. The Python environment is whatever interpreter runs this
tool unless ``anaconda`` names a conda environment root.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
from dataclasses import dataclass
from typing import Any, Dict

import yaml

from .config import dataclass_from_dict, from_cli, load_yaml


@dataclass
class StoolArgs:
    config: Any = None
    launcher: str = "sbatch"  # "sbatch" submits; "bash" runs inside an allocation
    script: str = "apps.main.train"  # module run by every task
    copy_code: bool = True  # snapshot the code into dump_dir/code and run from there
    dirs_exists_ok: bool = False
    override: bool = False  # delete an existing dump_dir first (asks for confirmation)
    nodes: int = -1
    ngpu: int = 8  # GPUs (= tasks) per node
    ncpu: int = 16  # CPUs per GPU
    mem: str = ""
    anaconda: str = "default"  # conda env root, or "default" for the current interpreter
    constraint: str = ""
    exclude: str = ""
    time: int = -1  # minutes; -1 = the partition's maximum
    account: str = ""
    qos: str = ""
    partition: str = "learn"
    stdout: bool = False


SBATCH_COMMAND = """#!/bin/bash
{exclude}
{qos}
{account}
{constraint}
#SBATCH --job-name={name}
#SBATCH --nodes={nodes}
#SBATCH --gres=gpu:{ngpus}
#SBATCH --cpus-per-gpu={ncpu}
#SBATCH --time={time}
#SBATCH --partition={partition}
#SBATCH --mem={mem}
#SBATCH --output={dump_dir}/logs/%j/%j.stdout
#SBATCH --error={dump_dir}/logs/%j/%j.stderr
#SBATCH --open-mode=append
#SBATCH --signal=USR2@120
#SBATCH --distribution=block

{activate}
{go_to_code_dir}
export OMP_NUM_THREADS=1
export LAUNCH_WITH="SBATCH"
export DUMP_DIR={dump_dir}
srun {log_output} -n {tasks} -N {nodes_per_run} {python} -u -m {script} config=$DUMP_DIR/base_config.yaml
"""


def copy_dir(input_dir: str, output_dir: str) -> None:
    """Copy the ``*.py`` tree (and built kernel libraries) of ``input_dir``."""
    print(f"Copying : {input_dir}\nto      : {output_dir} ...")
    assert os.path.isdir(input_dir), f"{input_dir} is not a directory"
    assert os.path.isdir(output_dir), f"{output_dir} is not a directory"
    if shutil.which("rsync"):
        cmd = (f"rsync -arm --copy-links --include '**/' --include '*.py' --include '*.so' --include '*.cu' "
               f"--include '*.cuh' --include '*.h' --include '*.yaml' --exclude='*' {input_dir}/ {output_dir}")
        print(f"Copying command: {cmd}")
        subprocess.call([cmd], shell=True)
    else:
        keep = (".py", ".so", ".cu", ".cuh", ".h", ".yaml")
        for root, _dirs, files in os.walk(input_dir):
            if os.path.abspath(root).startswith(os.path.abspath(output_dir)):
                continue
            for f in files:
                if f.endswith(keep):
                    dst = os.path.join(output_dir, os.path.relpath(root, input_dir))
                    os.makedirs(dst, exist_ok=True)
                    shutil.copy2(os.path.join(root, f), dst)
    print("Copy done.")


def retrieve_max_time_per_partition() -> Dict[str, int]:
    sinfo = json.loads(subprocess.check_output("sinfo --json", shell=True))["sinfo"]
    out: Dict[str, int] = {}
    for info in sinfo:
        t = info["partition"]["maximums"]["time"]
        out[info["partition"]["name"]] = 14 * 24 * 60 if t["infinite"] else t["number"]
    return out


def validate_args(args: StoolArgs) -> None:
    if args.time == -1:
        try:
            args.time = retrieve_max_time_per_partition().get(args.partition, 3 * 24 * 60)
        except Exception:
            args.time = 3 * 24 * 60
        print(f"No time limit specified, using max time for partitions: {args.time} minutes")
    if args.constraint:
        args.constraint = f"#SBATCH --constraint={args.constraint}"
    if args.account:
        args.account = f"#SBATCH  --account={args.account}"
    if args.qos:
        args.qos = f"#SBATCH --qos={args.qos}"
    if args.exclude:
        args.exclude = f"#SBATCH --exclude={args.exclude}"
    if args.anaconda:
        args.anaconda = sys.executable if args.anaconda == "default" else f"{args.anaconda}/bin/python"
        assert os.path.isfile(args.anaconda)
    args.mem = args.mem or "0"
    assert args.partition
    assert args.ngpu > 0 and args.ncpu > 0 and args.nodes > 0 and args.time > 0


def launch_job(args: StoolArgs) -> None:
    validate_args(args)
    dump_dir, job_name = args.config["dump_dir"], args.config["name"]
    print("Creating directories...")
    os.makedirs(dump_dir, exist_ok=args.dirs_exists_ok or args.override)
    if args.override:
        confirm = input(f"Are you sure you want to delete the directory '{dump_dir}'? "
                        f"This action cannot be undone. (yes/no): ")
        if confirm.lower() != "yes":
            print("Operation cancelled.")
            return
        shutil.rmtree(dump_dir)
        os.makedirs(dump_dir)
        print(f"Directory '{dump_dir}' has been deleted.")
    if args.copy_code:
        os.makedirs(f"{dump_dir}/code", exist_ok=args.dirs_exists_ok)
        print("Copying code ...")
        copy_dir(os.getcwd(), f"{dump_dir}/code")
    print("Saving config file ...")
    with open(f"{dump_dir}/base_config.yaml", "w") as f:
        yaml.safe_dump(args.config, f, sort_keys=False)
    conda_exe = os.environ.get("CONDA_EXE")
    activate = ""
    if conda_exe and args.anaconda != sys.executable:
        env_path = os.path.dirname(os.path.dirname(args.anaconda))
        activate = f'eval "$({conda_exe} shell.bash hook)"\nsource activate {env_path}'
    log_output = "" if args.stdout else "-o $DUMP_DIR/logs/%j/%j_%t.out -e $DUMP_DIR/logs/%j/%j_%t.err"
    sbatch = SBATCH_COMMAND.format(
        name=job_name, script=args.script, dump_dir=dump_dir, nodes=args.nodes, tasks=args.nodes * args.ngpu,
        nodes_per_run=args.nodes, ngpus=args.ngpu, ncpu=args.ncpu, mem=args.mem, qos=args.qos, account=args.account,
        constraint=args.constraint, exclude=args.exclude, time=args.time, partition=args.partition,
        activate=activate, python=args.anaconda or "python", log_output=log_output,
        go_to_code_dir=f"cd {dump_dir}/code/" if args.copy_code else "")
    print("Writing sbatch command ...")
    with open(f"{dump_dir}/submit.slurm", "w") as f:
        f.write(sbatch)
    print("Submitting job ...")
    os.system(f"{args.launcher} {dump_dir}/submit.slurm")
    print("Done.")


if __name__ == "__main__":
    cli = from_cli()
    cli["config"] = load_yaml(cli["config"])
    launch_job(dataclass_from_dict(StoolArgs, cli))
