"""Shared helpers for the parity tests: compare table lookups with oracle puts."""
import numpy as np

import oracle_lib


def split_keys(keys, key_off):
    kb = keys.tobytes()
    return [kb[int(key_off[i]):int(key_off[i + 1])] for i in range(len(key_off) - 1)]


def compare_puts(db, keys, key_off, rect, dec, corners=("hi", "lo"), chunk=200000):
    """Every oracle put says: the whole rectangle [lo..hi] of the limits lattice has decision
    `dec`. Check the GPU table at the rectangle's corners. Returns a list of mismatch strings."""
    blobs = split_keys(keys, key_off)
    bad = []
    for corner in corners:
        codes = rect[:, 4:] if corner == "hi" else rect[:, :4]
        limits = oracle_lib.codes_to_limits(codes)
        for lo in range(0, len(blobs), chunk):
            hi = min(len(blobs), lo + chunk)
            got = db.get_many(blobs[lo:hi], limits[lo:hi].tolist())
            for i, g in enumerate(got):
                want = dec[lo + i]
                if g.found == -1:
                    bad.append(f"{corner} #{lo + i}: Spec missing from the GPU tables")
                elif g.found != int(want["found"]):
                    bad.append(f"{corner} #{lo + i}: found {g.found} != {int(want['found'])}")
                elif g.found == 1 and (g.action != int(want["action"]) or g.main_cost != int(want["main"]) or
                                       g.depth != int(want["depth"]) or
                                       tuple(g.peaks) != tuple(int(x) for x in want["peaks"])):
                    bad.append(f"{corner} #{lo + i}: got {g} want {want}")
                if len(bad) > 20:
                    return bad
    return bad
