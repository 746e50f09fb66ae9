#!/usr/bin/env python3
"""Pins the range-expansion oracle to the REAL reference library.

TEST INFRASTRUCTURE ONLY.

The command handler of the reference preload library is a static function that
only runs inside a live CUDA process.  This script builds the unmodified
``select.cpp`` (``make -C oracle ref``), preloads it into a small driver program
together with a stub CUDA driver and a stub NVML, lets the program allocate
"device" memory, sends plan commands through the library's real control
socket, and records the replies and the cuMemPrefetchAsync calls each plan
produced.  The result is committed as ``tests/golden/reference_uvm_socket.json``;
``tests/test_reference_socket_golden.py`` holds the oracle, the C++ expander
and the UVM server of this repository to it.

    python oracle/drive_ref.py [/path/to/reference]

Needs the reference checkout; the tests only need the committed fixture.
"""
import json
import os
import random
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
MIB = 1 << 20
BIG = (1 << 64) - 1


def run(lib: Path, sizes, commands, chunk_mb=16):
    """Returns {allocs: [...], results: [{line, reply, status, calls}]}."""
    env = dict(os.environ, SELECT_UVM_ENABLE="1", SELECT_UVM_CONVERT_ALLOC="1",
               SELECT_UVM_CHUNK_MB=str(chunk_mb), LD_PRELOAD=str(lib),
               LD_LIBRARY_PATH=str(HERE / "_ref" / "stubs"),
               RETARGET_B200_LIBCUDA=str(HERE / "_ref" / "stubs" / "libcuda.so"))
    out = subprocess.run([str(HERE / "_ref" / "drive_app"), str(HERE / "_ref" / "stubs" / "libcuda.so"),
                          *map(str, sizes)], input="".join(c + "\n" for c in commands).encode(), env=env,
                         capture_output=True, timeout=600)
    stdout = out.stdout.decode()          # bytes mode: a command may contain a carriage return
    allocs, results, cur, next_id = [], [], None, 1
    for line in stdout.split("\n"):
        if line.startswith("ALLOC "):
            _, idx, size, _, rc, ptr = line.split()
            assert rc == "0", line
            allocs.append(dict(id=next_id, bytes=int(size), ptr=int(ptr, 16), device=0, concurrent=1))
            next_id += 1
        elif line.startswith("FREE "):
            idx = int(line.split()[1])
            allocs = [a for a in allocs if a["id"] != idx]
        elif line.startswith("REPLY "):
            cmd, _, body = line[6:].partition(" -> ")
            cur = dict(line=cmd, reply=json.loads(body), calls=[])
            results.append(cur)
        elif line.startswith("STATUS "):
            cur["status"] = json.loads(line[7:])
        elif line.startswith("CALL prefetch "):
            _, _, ptr, nbytes, dst, _stream = line.split()
            ptr = int(ptr, 16)
            a = next(x for x in allocs if x["ptr"] <= ptr < x["ptr"] + x["bytes"])
            cur["calls"].append([a["id"], ptr - a["ptr"], int(nbytes), int(dst)])
    assert len(results) == len(commands), (len(results), len(commands), stdout[-2000:], out.stderr[-2000:])
    return dict(allocs=[{k: a[k] for k in ("id", "bytes", "device", "concurrent")} for a in allocs],
                results=results)


def fixed_commands(gen, A, n, other_id):
    return [
        "status", "list",
        f"windowv {gen} {A} {n} {BIG} {BIG} 0 {8 * MIB}",
        f"windowv {gen} {A} {n} 0 {8 * MIB} {2 * MIB} {10 * MIB}",
        f"windowv {gen} {A} {n} {2 * MIB} {10 * MIB} {20 * MIB} {28 * MIB}",
        f"windowv {gen} {A} {n} {20 * MIB} {28 * MIB} {4 * MIB} {30 * MIB}",
        f"windowv {gen} {A} {n} {4 * MIB} {30 * MIB} {4 * MIB} {30 * MIB}",
        f"windowfullv {gen} {A} {n} {4 * MIB} {30 * MIB} {24 * MIB} {A}",
        f"windowfullv {gen} {A} {n} {BIG} {BIG} 0 {A}",
        f"blocksv {gen} {A} {n} {2 * MIB} f00f1",
        f"blocksv {gen} {A} {n} {2 * MIB} ffff",
        f"blocksv {gen} {A} {n} {2 * MIB} 8000",
        f"blocksv {gen} {A} {n} {2 * MIB} 5555",
        f"blocksv {gen} {A} {n} {3 * MIB} 7ff",
        f"blocksv {gen} {A} {n} {3 * MIB} 400",
        f"blocksv {gen} {A} {n} {5 * MIB + 4096} 7f",
        f"blocksv {gen} {A} {n} {A} 1",
        f"blocksv {gen} {A} {n} 4096 " + "f" * 256,
        f"prefetch {other_id} 0 4096 cpu", f"prefetch {other_id} 0 4096 gpu",
        f"prefetch 1 {4 * MIB} {40 * MIB} gpu",
        f"target {40 * MIB}", f"target 0", f"targetv {gen} {70 * MIB}",
        f"retarget {gen} {40 * MIB} {70 * MIB}", f"retarget {gen} {70 * MIB} {8 * MIB}",
        f"retarget {gen} {8 * MIB} {8 * MIB}",
        # rejections
        "bogus", "", "status now", f"windowv {gen + 1} {A} {n} 0 0 0 {MIB}",
        f"windowv {gen} {A} {n + 1} 0 0 0 {MIB}", f"windowv {gen} {A} {n} 0 0 5 {MIB}",
        f"windowv {gen} {A} {n} 0 0 {2 * MIB} {MIB}", f"windowv {gen} {A} {n} 0 0 0 {A + 4096}",
        f"windowv {gen} 0 {n} 0 0 0 0", f"windowv {gen} {A} 0 0 0 0 0",
        f"windowv {gen} {A} {n} 7 {MIB} 0 {MIB}", f"windowv {gen} {A} {n} {BIG} 0 0 {MIB}",
        f"blocksv {gen} {A} {n} {2 * MIB} 0", f"blocksv {gen} {A} {n} {2 * MIB} 10000",
        f"blocksv {gen} {A} {n} {2 * MIB} xyz", f"blocksv {gen} {A} {n} {2 * MIB} F",
        f"blocksv {gen} {A} {n} 123 1", f"blocksv {gen} {A} {n} 0 1", f"blocksv {gen} {A} {n} {2 * A} 1",
        f"blocksv {gen} {A} 0 {2 * MIB} 1", f"blocksv {gen + 3} {A} {n} {2 * MIB} 1",
        f"blocksv {gen} {A} {n} {2 * MIB} " + "1" * 257, f"blocksv {gen} {A} {n + 2} {2 * MIB} 1",
        "prefetch 999 0 4096 gpu", f"prefetch {other_id} 4096 0 gpu", f"prefetch {other_id} 100 4096 gpu",
        f"prefetch {other_id} 0 100 gpu", f"prefetch {other_id} 0 8192 gpu", f"prefetch 1 0 4096 tpu",
        f"target {1 << 50}", "target 100", "target 18446744073709551616", "target -1", "target 1\t",
        f"targetv {gen + 1} 0", f"retarget {gen} 100 0", f"retarget {gen} 0 {1 << 50}",
        f"retarget {gen + 1} 0 0", "\ttarget\r 4096 ", f"windowv\t{gen} {A} {n} 0 0 0 4096",
        "1 2 3 4 5 6 7 8 9",
    ]


def fuzz_commands(rng, gen, A, n, allocs, count):
    managed = sum(a["bytes"] for a in allocs)
    page = 4096
    out = []
    for _ in range(count):
        kind = rng.choice(["blocksv", "windowv", "windowfullv", "target", "targetv", "retarget", "prefetch"])
        g = gen if rng.random() > .05 else gen + 1
        k = n if rng.random() > .05 else n + 1
        if kind == "blocksv":
            blk = rng.choice([page, 2 * MIB, 512 * 1024, 3 * MIB, A])
            nb = -(-A // blk)
            if nb > 1024:
                blk, nb = 2 * MIB, -(-A // (2 * MIB))
            bits = [b for b in range(nb) if rng.random() < rng.choice([0.05, 0.5, 0.95])]
            mask = format(sum(1 << b for b in bits), "x")
            if rng.random() < .05:
                mask += "0"
            out.append(f"blocksv {g} {A} {k} {blk} {mask}")
        elif kind in ("windowv", "windowfullv"):
            def edge():
                return min(A, rng.randint(0, A // MIB) * MIB + rng.choice([0, 0, 0, 1, page]))
            o, w = sorted([edge(), edge()]), sorted([edge(), edge()])
            if rng.random() < .2:
                o = [BIG, BIG]
            if rng.random() < .1:
                w[1] = A
            out.append(f"{kind} {g} {A} {k} {o[0]} {o[1]} {w[0]} {w[1]}")
        elif kind == "target":
            out.append(f"target {rng.choice([0, managed, rng.randint(0, managed) // page * page, rng.randint(0, managed + 9)])}")
        elif kind == "targetv":
            out.append(f"targetv {g} {rng.randint(0, managed) // page * page}")
        elif kind == "retarget":
            out.append(f"retarget {g} {rng.randint(0, managed) // page * page} "
                       f"{rng.choice([0, managed, rng.randint(0, managed) // page * page])}")
        else:
            a = rng.choice(allocs)
            off = rng.choice([0, page, rng.randint(0, a["bytes"]) // page * page, rng.randint(0, a["bytes"])])
            ln = rng.choice([page, max(0, a["bytes"] - off), rng.randint(0, a["bytes"]) // page * page])
            out.append(f"prefetch {a['id'] + rng.choice([0, 0, 0, 500])} {off} {ln} {rng.choice(['cpu', 'gpu'])}")
    return out


def scenarios():
    rng = random.Random(2024)
    A = 32 * MIB
    s1_sizes = [A, A, 4096, A, 12345 * 4096, A]
    s1_allocs = [dict(id=i + 1, bytes=b) for i, b in enumerate(s1_sizes)]
    yield dict(name="six allocations, four cache buffers of 32 MiB", sizes=s1_sizes, chunk_mb=16,
               commands=fixed_commands(6, A, 4, 3) + fuzz_commands(rng, 6, A, 4, s1_allocs, 220))
    # allocation that is not a multiple of the block: partial last block; one allocation freed
    B = 7 * MIB + 8192
    s2_sizes = [B, 64 * 1024, B, B, "-2", 4096]
    s2_allocs = [dict(id=1, bytes=B), dict(id=3, bytes=B), dict(id=4, bytes=B), dict(id=5, bytes=4096)]
    cmds = [f"blocksv 6 {B} 3 {2 * MIB} f", f"blocksv 6 {B} 3 {2 * MIB} 8", f"blocksv 6 {B} 3 {2 * MIB} 9",
            f"blocksv 6 {B} 3 {2 * MIB} 10", f"windowv 6 {B} 3 {BIG} {BIG} {MIB} {B}",
            f"windowv 6 {B} 3 {MIB} {B} 0 {3 * MIB}", "list"]
    yield dict(name="7 MiB + 8 KiB buffers (partial last block), one allocation freed", sizes=s2_sizes,
               chunk_mb=1, commands=cmds + fuzz_commands(rng, 6, B, 3, s2_allocs, 120))


def main():
    reference = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["RETARGET_REFERENCE"])
    subprocess.run(["make", "-C", str(HERE), "ref", f"REFERENCE={reference}"], check=True, capture_output=True)
    doc = dict(generated_by="oracle/drive_ref.py: unmodified select.cpp driven through its own socket under "
                            "a stub CUDA driver", scenarios=[])
    for sc in scenarios():
        got = run(HERE / "_ref" / "libselect_ref.so", sc["sizes"], sc["commands"], sc["chunk_mb"])
        doc["scenarios"].append(dict(name=sc["name"], sizes=sc["sizes"], chunk_mb=sc["chunk_mb"], **got))
        errors = sum(1 for r in got["results"] if not r["reply"].get("ok"))
        print(sc["name"], len(got["results"]), "commands,", errors, "rejected,",
              sum(len(r["calls"]) for r in got["results"]), "prefetch calls")
    path = ROOT / "tests" / "golden" / "reference_uvm_socket.json"
    path.write_text(json.dumps(doc, separators=(",", ":")))
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
