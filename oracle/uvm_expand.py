"""Oracle: plan-command parsing and range expansion of the preload library.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

Restates the command handler of the reference's UVM control socket
(select.cpp:24045-24327): word splitting, unsigned parsing, validation order
with its error strings, and the (allocation id, offset, bytes, destination)
range list each accepted plan produces.  The registry is a list of dicts
``{"id", "bytes", "device", "concurrent"}`` in insertion order
(select.cpp:23770-23778).

The handler is a ``static`` function of a library that only acts inside a live
CUDA process, so it cannot be called directly; ``oracle/Makefile`` builds the
reference library and ``oracle/drive_ref.py`` drives it through its real socket
under a stub driver.  The recorded replies and prefetch calls pin this file
(tests/test_reference_socket_golden.py).
"""
from __future__ import annotations

CPU = -1                      # CU_DEVICE_CPU
UINT64_MAX = (1 << 64) - 1
PAGE = 4096                   # sysconf(_SC_PAGESIZE) on the supported hosts


class PlanError(Exception):
    """Carries the error string the socket would send back."""


def parse_uint(word: str) -> int:
    """Unsigned decimal with overflow check (select.cpp:23826-23837)."""
    if not word:
        raise PlanError("invalid_command")
    n = 0
    for ch in word:
        if ch < "0" or ch > "9":
            raise PlanError("invalid_command")
        d = ord(ch) - 48
        if n > (UINT64_MAX - d) // 10:
            raise PlanError("invalid_command")
        n = n * 10 + d
    return n


def split_words(line: str):
    """Space/tab/CR separated, at most eight words (select.cpp:24047-24054)."""
    words = [w for w in line.replace("\t", " ").replace("\r", " ").split(" ") if w]
    if not words or len(words) > 8:
        raise PlanError("invalid_command")
    return words


def _emit(out, alloc, offset, nbytes, device):
    """Zero-length ranges are dropped (select.cpp:23924-23937)."""
    if nbytes:
        out.append((alloc["id"], offset, nbytes, device))


def expand_blocks(registry, generation, *, gen, alloc_bytes, count, block_bytes, mask,
                  page=PAGE):
    """``blocksv`` (select.cpp:24147-24195).  In the C++ the variable called
    ``block`` holds the allocation size and ``bytes`` the block size."""
    digits = len(mask)
    if gen != generation:
        raise PlanError("stale_allocations")
    if (not alloc_bytes or not block_bytes or block_bytes > alloc_bytes
            or block_bytes % page or not count):
        raise PlanError("invalid_block_geometry")
    if not digits or digits > 256:
        raise PlanError("invalid_block_mask")
    n_blocks = alloc_bytes // block_bytes + (alloc_bytes % block_bytes != 0)
    any_bit = False
    error = None
    for d in range(digits):
        ch = mask[digits - 1 - d]
        if "0" <= ch <= "9":
            value = ord(ch) - 48
        elif "a" <= ch <= "f":
            value = ord(ch) - 87
        else:
            raise PlanError("invalid_block_mask")
        for bit in range(4):
            if value & (1 << bit):
                any_bit = True
                if d * 4 + bit >= n_blocks:
                    error = "block_out_of_range"
        if error:
            # the C loop stops at the first digit that set an error
            break
    if error:
        raise PlanError(error)
    if not any_bit:
        raise PlanError("empty_block_mask")
    matched = 0
    for a in registry:
        if a["bytes"] != alloc_bytes:
            continue
        matched += 1
        if not a["concurrent"]:
            raise PlanError("concurrent_managed_access_required")
    if matched != count:
        raise PlanError("cache_allocation_count_mismatch")
    bits = int(mask, 16)
    out = []
    whole = alloc_bytes // block_bytes
    for a in registry:
        if a["bytes"] != alloc_bytes:
            continue
        begin = None
        for index in range(n_blocks + 1):
            chosen = index < n_blocks and (index // 4) < digits and (bits >> index) & 1
            if chosen and begin is None:
                begin = index
            if not chosen and begin is not None:
                end = alloc_bytes if index > whole else index * block_bytes
                _emit(out, a, begin * block_bytes, end - begin * block_bytes, a["device"])
                begin = None
    return out


def expand_window(registry, generation, *, gen, alloc_bytes, count, old, new,
                  full_refresh: bool, page=PAGE):
    """``windowv`` / ``windowfullv`` (select.cpp:24196-24249): every range that
    moves to the CPU precedes every range that moves to the GPU."""
    ob, oe = old
    nb, ne = new
    initial = ob == UINT64_MAX and oe == UINT64_MAX
    if gen != generation:
        raise PlanError("stale_allocations")
    if (not alloc_bytes or not count or nb > ne or ne > alloc_bytes
            or nb % page or (ne != alloc_bytes and ne % page)
            or (not initial and (ob > oe or oe > alloc_bytes or ob % page
                                 or (oe != alloc_bytes and oe % page)))):
        raise PlanError("invalid_window")
    matched = 0
    for a in registry:
        if a["bytes"] == alloc_bytes:
            matched += 1
        if (initial or a["bytes"] == alloc_bytes) and not a["concurrent"]:
            raise PlanError("concurrent_managed_access_required")
    if matched != count:
        raise PlanError("cache_allocation_count_mismatch")
    out = []
    for phase in (0, 1):
        for a in registry:
            if a["bytes"] != alloc_bytes:
                if initial and phase:
                    _emit(out, a, 0, a["bytes"], a["device"])
                continue
            if initial or full_refresh:
                spans = ([(0, nb), (ne, alloc_bytes)] if not phase else [(nb, ne)])
            else:
                sb, se = (nb, ne) if phase else (ob, oe)
                tb, te = (ob, oe) if phase else (nb, ne)
                spans = [(sb, min(se, tb)), (max(sb, te), se)]
            for lo, hi in spans:
                if hi > lo:
                    _emit(out, a, lo, hi - lo, a["device"] if phase else CPU)
    return out


def expand_prefetch(registry, *, alloc_id, offset, nbytes, where, page=PAGE):
    """``prefetch`` (select.cpp:24136-24146)."""
    a = next((x for x in registry if x["id"] == alloc_id), None)
    if a is None:
        raise PlanError("unknown_id")
    if not nbytes or offset >= a["bytes"] or nbytes > a["bytes"] - offset:
        raise PlanError("invalid_range")
    if offset % page or (nbytes % page and nbytes != a["bytes"] - offset):
        raise PlanError("unaligned_range")
    if not a["concurrent"]:
        raise PlanError("concurrent_managed_access_required")
    out = []
    _emit(out, a, offset, nbytes, CPU if where == "cpu" else a["device"])
    return out


def _check_prefix(registry, target, page):
    """Alignment walk shared by target/targetv/retarget (select.cpp:24257-24263,
    24288-24293)."""
    remaining = target
    for a in registry:
        gpu = min(remaining, a["bytes"])
        remaining -= gpu
        if gpu != a["bytes"] and gpu % page:
            raise PlanError("unaligned_target")
        if not a["concurrent"]:
            raise PlanError("concurrent_managed_access_required")


def expand_target(registry, generation, *, nbytes, gen=None, page=PAGE):
    """``target`` / ``targetv`` (select.cpp:24281-24309)."""
    managed = sum(a["bytes"] for a in registry)
    if gen is not None and gen != generation:
        raise PlanError("stale_allocations")
    if nbytes > managed:
        raise PlanError("target_exceeds_managed_bytes")
    _check_prefix(registry, nbytes, page)
    out = []
    for phase in (0, 1):
        remaining = nbytes
        for a in registry:
            gpu = min(remaining, a["bytes"])
            remaining -= gpu
            if phase:
                _emit(out, a, 0, gpu, a["device"])
            else:
                _emit(out, a, gpu, a["bytes"] - gpu, CPU)
    return out


def expand_retarget(registry, generation, *, gen, old, new, page=PAGE):
    """``retarget`` (select.cpp:24250-24280)."""
    managed = sum(a["bytes"] for a in registry)
    if gen != generation:
        raise PlanError("stale_allocations")
    if old > managed or new > managed:
        raise PlanError("target_exceeds_managed_bytes")
    _check_prefix(registry, old, page)
    _check_prefix(registry, new, page)
    out = []
    if old != new:
        lower, upper = min(old, new), max(old, new)
        base = 0
        for a in registry:
            end = base + a["bytes"]
            lo, hi = max(lower, base), min(upper, end)
            if hi > lo:
                _emit(out, a, lo - base, hi - lo, a["device"] if new > old else CPU)
            base = end
    return out


def command(registry, generation, line: str, page=PAGE):
    """Full handler for a plan line: returns the range list or raises PlanError
    with the string the socket would report.  ``status`` and ``list`` are
    answered by the server itself and are not plans."""
    words = split_words(line)
    name, n = words[0], len(words)
    if name == "blocksv" and n == 6:
        gen, a, c, b = (parse_uint(w) for w in words[1:5])
        return expand_blocks(registry, generation, gen=gen, alloc_bytes=a, count=c,
                             block_bytes=b, mask=words[5], page=page)
    if name in ("windowv", "windowfullv") and n == 8:
        v = [parse_uint(w) for w in words[1:8]]
        return expand_window(registry, generation, gen=v[0], alloc_bytes=v[1], count=v[2],
                             old=(v[3], v[4]), new=(v[5], v[6]),
                             full_refresh=name == "windowfullv", page=page)
    if name == "prefetch" and n == 5:
        i, o, b = (parse_uint(w) for w in words[1:4])
        if words[4] not in ("cpu", "gpu"):
            raise PlanError("invalid_command")
        return expand_prefetch(registry, alloc_id=i, offset=o, nbytes=b, where=words[4], page=page)
    if name == "target" and n == 2:
        return expand_target(registry, generation, nbytes=parse_uint(words[1]), page=page)
    if name == "targetv" and n == 3:
        return expand_target(registry, generation, gen=parse_uint(words[1]),
                             nbytes=parse_uint(words[2]), page=page)
    if name == "retarget" and n == 4:
        g, o, w = (parse_uint(x) for x in words[1:4])
        return expand_retarget(registry, generation, gen=g, old=o, new=w, page=page)
    raise PlanError("invalid_command")
