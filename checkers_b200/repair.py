"""Command-line front end of the prefix-mask Re-Pair size estimator.

    python -m checkers_b200.repair <export_dir> [--state-type NAME] [--category NAME]
           [--group-id N] [--max-rules N] [--masked-mantissa-bits N] [--device N]

Same arguments, inputs and report files as the reference's stand-alone tool
(src/tensor_group_prefix_mask_repair.cpp in the Checkers tree; argument parsing
:600-626, driver :628-741): it reads <export_dir>/manifest.csv and
<export_dir>/analysis/plots/grouping_summary.csv plus the raw tensor files they
name, and writes under <export_dir>/prefix_mask_repair/
    tensor_prefix_mask_repair.csv, group_prefix_mask_repair.csv,
    checkpoint_prefix_mask_repair_summary.txt
The pair counting and sequence rewriting run on the GPU (chk_repair_build /
chk_repair_apply); this file is file handling, size accounting (:653-655,
:686-712) and the report text (:477-598).  Numbers are formatted the way C++
streams format them (default precision for the CSV files, fixed 6 digits for
the summary) so the reports compare equal apart from the time columns.
"""
import ctypes as C
import os
import sys
import time

import numpy as np

from ._lib import lib

MB = 1024.0 * 1024.0
LAYOUTS = {"float32": (4, 23), "float16": (2, 10), "fp16": (2, 10), "bfloat16": (2, 7), "bf16": (2, 7)}

lib.chk_repair_last_error.restype = C.c_char_p
_u32p, _u64p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
lib.chk_repair_build.restype = C.c_int
lib.chk_repair_build.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, _u32p, _u32p, _u64p,
                                 _u32p, _u64p, _u64p, _u64p]
lib.chk_repair_apply.restype = C.c_int
lib.chk_repair_apply.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, _u32p, _u32p, C.c_uint32, _u64p]


class RepairError(RuntimeError):
    pass


def _check(rc):
    if rc != 0:
        raise RepairError(f"[checkers_b200.repair] error {rc}: {lib.chk_repair_last_error().decode(errors='replace')}")


def build_grammar(raw, storage_bytes, masked_bits, max_rules, device=0):
    """Grammar of one tensor (uint8 array of its bytes).  Returns a dict with the rules as
    token ids, the rewritten length, the largest pair count seen and the number of tie rounds."""
    raw = np.ascontiguousarray(raw, np.uint8)
    numel = raw.size // storage_bytes
    lhs, rhs = np.zeros(max(max_rules, 1), np.uint32), np.zeros(max(max_rules, 1), np.uint32)
    freq = np.zeros(max(max_rules, 1), np.uint64)
    n_rules, tokens, max_freq, ties = C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint64()
    _check(lib.chk_repair_build(device, raw.ctypes.data, numel, storage_bytes, masked_bits, max_rules,
                                lhs.ctypes.data_as(_u32p), rhs.ctypes.data_as(_u32p), freq.ctypes.data_as(_u64p),
                                C.byref(n_rules), C.byref(tokens), C.byref(max_freq), C.byref(ties)))
    k = n_rules.value
    return dict(lhs=lhs[:k].copy(), rhs=rhs[:k].copy(), freq=freq[:k].copy(), tokens=tokens.value,
                max_pair_frequency=max_freq.value, tie_rounds=ties.value)


def apply_grammar(raw, storage_bytes, masked_bits, lhs, rhs, device=0):
    raw = np.ascontiguousarray(raw, np.uint8)
    lhs, rhs = np.ascontiguousarray(lhs, np.uint32), np.ascontiguousarray(rhs, np.uint32)
    tokens = C.c_uint64()
    _check(lib.chk_repair_apply(device, raw.ctypes.data, raw.size // storage_bytes, storage_bytes, masked_bits,
                                lhs.ctypes.data_as(_u32p), rhs.ctypes.data_as(_u32p), lhs.size, C.byref(tokens)))
    return tokens.value


# ---------------------------------------------------------------- text helpers
def split_csv_row(line):
    cols, cur, quoted = [], [], False
    for ch in line:
        if ch == '"':
            quoted = not quoted
        elif ch == "," and not quoted:
            cols.append("".join(cur))
            cur = []
        else:
            cur.append(ch)
    cols.append("".join(cur))
    return [c.strip(" \t\r") for c in cols]


def g6(x):
    """A double as `std::ostream << x` prints it with default settings (%g, 6 significant digits)."""
    return "%g" % x


def f6(x):
    return "%.6f" % x


def bits_to_bytes(bits):
    return (bits + 7) // 8


def ratio(a, b):
    return 0.0 if abs(b) <= sys.float_info.epsilon else a / b


def token_width(symbol_count):
    if symbol_count <= 1:
        return 1
    return max((symbol_count - 1).bit_length(), 1)


def read_manifest(path):
    entries = {}
    with open(path) as f:
        f.readline()
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            c = split_csv_row(line)
            if len(c) != 7:
                raise RepairError("Malformed manifest row: " + line)
            entries[(c[3], c[2], int(c[1]))] = dict(key=c[0], layer=int(c[1]), category=c[2], state_type=c[3],
                                                    numel=int(c[4]), dtype=c[5],
                                                    path=os.path.join(os.path.dirname(path), c[6]))
    return entries


def read_groups(path, state_type=None, category=None, group_id=None):
    groups = []
    with open(path) as f:
        f.readline()
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            c = split_csv_row(line)
            if len(c) < 10:
                raise RepairError("Malformed grouping summary row: " + line)
            g = dict(state_type=c[0], category=c[1], group_id=int(c[2]), layers=[int(t) for t in c[4].split()],
                     representative=int(c[5]))
            if state_type is not None and g["state_type"] != state_type:
                continue
            if category is not None and g["category"] != category:
                continue
            if group_id is not None and g["group_id"] != group_id:
                continue
            groups.append(g)
    return groups


def load_tensor(entry, storage_bytes):
    want = entry["numel"] * storage_bytes
    raw = np.fromfile(entry["path"], dtype=np.uint8, count=want)
    if raw.size != want:
        raise RepairError("Tensor payload size mismatch: " + entry["path"])
    return raw


def run(export_dir, state_type=None, category=None, group_id=None, max_rules=50, masked_mantissa_bits=None, device=0):
    manifest = read_manifest(os.path.join(export_dir, "manifest.csv"))
    groups = read_groups(os.path.join(export_dir, "analysis", "plots", "grouping_summary.csv"), state_type, category,
                         group_id)
    if not groups:
        raise RepairError("No matching grouping rows found for the requested filters")
    out_dir = os.path.join(export_dir, "prefix_mask_repair")
    os.makedirs(out_dir, exist_ok=True)

    tensor_rows, group_rows, tie_rounds = [], [], 0
    for g in groups:
        rep = manifest.get((g["state_type"], g["category"], g["representative"]))
        if rep is None:
            raise RepairError("Missing representative tensor in manifest for requested group")
        if rep["dtype"] not in LAYOUTS:
            raise RepairError("Unsupported dtype for mantissa-mask compression: " + rep["dtype"])
        storage, mantissa = LAYOUTS[rep["dtype"]]
        masked = min(mantissa if masked_mantissa_bits is None else masked_mantissa_bits, mantissa)
        remaining = storage * 8 - masked
        grammar = build_grammar(load_tensor(rep, storage), storage, masked, max_rules, device)
        tie_rounds += grammar["tie_rounds"]
        n_rules = len(grammar["lhs"])
        width = token_width((1 << remaining) + n_rules)
        grammar_bytes = bits_to_bytes(width * 2 * n_rules)
        gs = dict(g, dtype=rep["dtype"], masked=masked, rules=n_rules, grammar_bytes=grammar_bytes,
                  max_pair_frequency=grammar["max_pair_frequency"], original=0, masked_only=0, payload=0, residual=0,
                  lossy=0, time_ms=0.0)
        charged = False
        for layer in g["layers"]:
            t = manifest.get((g["state_type"], g["category"], layer))
            if t is None:
                raise RepairError("Missing grouped tensor in manifest")
            if t["dtype"] != rep["dtype"]:
                raise RepairError("Mixed dtypes inside one group are not supported")
            t0 = time.perf_counter()
            raw = load_tensor(t, storage)
            tokens = grammar["tokens"] if layer == g["representative"] else \
                apply_grammar(raw, storage, masked, grammar["lhs"], grammar["rhs"], device)
            payload = bits_to_bytes(width * tokens)
            charge = 0 if charged else grammar_bytes
            charged = True
            row = dict(state_type=g["state_type"], category=g["category"], group_id=g["group_id"], layer=layer,
                       rep=int(layer == g["representative"]), dtype=t["dtype"], numel=t["numel"], masked=masked,
                       original=t["numel"] * storage, masked_only=bits_to_bytes(t["numel"] * remaining), payload=payload,
                       charge=charge, lossy=payload + charge, residual=bits_to_bytes(t["numel"] * masked), tokens=tokens,
                       rules=n_rules, time_ms=(time.perf_counter() - t0) * 1e3)
            tensor_rows.append(row)
            for k_src, k_dst in (("original", "original"), ("masked_only", "masked_only"), ("payload", "payload"),
                                 ("residual", "residual"), ("lossy", "lossy")):
                gs[k_dst] += row[k_src]
            gs["time_ms"] += row["time_ms"]
        group_rows.append(gs)

    with open(os.path.join(out_dir, "tensor_prefix_mask_repair.csv"), "w") as f:
        f.write("state_type,category,group_id,layer,is_representative,dtype,numel,masked_mantissa_bits,original_size_mb,"
                "masked_only_size_mb,cfg_payload_size_mb,grammar_size_mb_charged,lossy_compressed_size_mb,"
                "residual_raw_size_mb,masking_only_ratio,compression_ratio,compressed_token_count,rule_count,time_ms\n")
        for r in tensor_rows:
            f.write(",".join([r["state_type"], r["category"], str(r["group_id"]), str(r["layer"]), str(r["rep"]),
                              r["dtype"], str(r["numel"]), str(r["masked"]), g6(r["original"] / MB),
                              g6(r["masked_only"] / MB), g6(r["payload"] / MB), g6(r["charge"] / MB), g6(r["lossy"] / MB),
                              g6(r["residual"] / MB), g6(ratio(r["original"], r["masked_only"])),
                              g6(ratio(r["original"], r["lossy"])), str(r["tokens"]), str(r["rules"]),
                              g6(r["time_ms"])]) + "\n")
    layers_text = lambda gs: " ".join(str(x) for x in gs["layers"])  # noqa: E731
    with open(os.path.join(out_dir, "group_prefix_mask_repair.csv"), "w") as f:
        f.write("state_type,category,group_id,layers,representative_layer,dtype,masked_mantissa_bits,rule_count,"
                "max_pair_frequency,original_group_size_mb,masked_only_group_size_mb,cfg_payload_group_size_mb,"
                "grammar_size_mb,lossy_compressed_group_size_mb,residual_raw_group_size_mb,masking_only_ratio,"
                "compression_ratio,total_time_ms\n")
        for gs in group_rows:
            f.write(",".join([gs["state_type"], gs["category"], str(gs["group_id"]), '"' + layers_text(gs) + '"',
                              str(gs["representative"]), gs["dtype"], str(gs["masked"]), str(gs["rules"]),
                              str(gs["max_pair_frequency"]), g6(gs["original"] / MB), g6(gs["masked_only"] / MB),
                              g6(gs["payload"] / MB), g6(gs["grammar_bytes"] / MB), g6(gs["lossy"] / MB),
                              g6(gs["residual"] / MB), g6(ratio(gs["original"], gs["masked_only"])),
                              g6(ratio(gs["original"], gs["lossy"])), g6(gs["time_ms"])]) + "\n")
    with open(os.path.join(out_dir, "checkpoint_prefix_mask_repair_summary.txt"), "w") as f:
        f.write("transform_mode: shared_group_mantissa_mask_cfg\n")
        f.write("state_type_filter: " + (state_type if state_type is not None else "<all>") + "\n")
        f.write("category_filter: " + (category if category is not None else "<all>") + "\n")
        f.write("group_id_filter: " + (str(group_id) if group_id is not None else "<all>") + "\n")
        f.write("masked_mantissa_bits_request: " +
                (str(masked_mantissa_bits) if masked_mantissa_bits is not None else "all_mantissa_bits") + "\n")
        f.write("max_rules_shared_grammar: " + str(max_rules) + "\n\n")
        tot = dict(original=0, masked_only=0, payload=0, lossy=0, residual=0, grammar_bytes=0)
        for gs in group_rows:
            for k in tot:
                tot[k] += gs[k]
            f.write(f"{gs['state_type']}/{gs['category']}/group_{gs['group_id']}: layers={layers_text(gs)}"
                    f", representative_layer={gs['representative']}, dtype={gs['dtype']}"
                    f", masked_mantissa_bits={gs['masked']}, rule_count={gs['rules']}"
                    f", original_group_size_mb={f6(gs['original'] / MB)}"
                    f", masked_only_group_size_mb={f6(gs['masked_only'] / MB)}"
                    f", cfg_payload_group_size_mb={f6(gs['payload'] / MB)}"
                    f", grammar_size_mb={f6(gs['grammar_bytes'] / MB)}"
                    f", lossy_compressed_group_size_mb={f6(gs['lossy'] / MB)}"
                    f", residual_raw_group_size_mb={f6(gs['residual'] / MB)}"
                    f", masking_only_ratio={f6(ratio(gs['original'], gs['masked_only']))}"
                    f", compression_ratio={f6(ratio(gs['original'], gs['lossy']))}\n")
        f.write("\nselected_groups_original_size_mb: " + f6(tot["original"] / MB) + "\n")
        f.write("selected_groups_masked_only_size_mb: " + f6(tot["masked_only"] / MB) + "\n")
        f.write("selected_groups_cfg_payload_size_mb: " + f6(tot["payload"] / MB) + "\n")
        f.write("selected_groups_total_grammar_mb: " + f6(tot["grammar_bytes"] / MB) + "\n")
        f.write("selected_groups_lossy_compressed_size_mb: " + f6(tot["lossy"] / MB) + "\n")
        f.write("selected_groups_residual_raw_size_mb: " + f6(tot["residual"] / MB) + "\n")
        f.write("selected_groups_masking_only_ratio: " + f6(ratio(tot["original"], tot["masked_only"])) + "\n")
        f.write("selected_groups_compression_ratio: " + f6(ratio(tot["original"], tot["lossy"])) + "\n")
    return dict(out_dir=out_dir, tie_rounds=tie_rounds, groups=len(group_rows), tensors=len(tensor_rows))


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        sys.stderr.write("Usage: python -m checkers_b200.repair <export_dir> [--state-type NAME] [--category NAME] "
                         "[--group-id N] [--max-rules N] [--masked-mantissa-bits N] [--device N]\n")
        return 1
    export_dir, kw, i = argv[0], {}, 1
    names = {"--state-type": ("state_type", str), "--category": ("category", str), "--group-id": ("group_id", int),
             "--max-rules": ("max_rules", int), "--masked-mantissa-bits": ("masked_mantissa_bits", int),
             "--device": ("device", int)}
    while i < len(argv):
        if argv[i] in names and i + 1 < len(argv):
            key, conv = names[argv[i]]
            kw[key] = conv(argv[i + 1])
            i += 2
        else:
            sys.stderr.write("Unknown or incomplete argument: " + argv[i] + "\n")
            return 1
    try:
        res = run(export_dir, **kw)
    except (RepairError, OSError, ValueError) as e:
        sys.stderr.write(str(e) + "\n")
        return 1
    base = res["out_dir"]
    print("Wrote tensor prefix-mask report to " + os.path.join(base, "tensor_prefix_mask_repair.csv"))
    print("Wrote group prefix-mask report to " + os.path.join(base, "group_prefix_mask_repair.csv"))
    print("Wrote prefix-mask summary to " + os.path.join(base, "checkpoint_prefix_mask_repair_summary.txt"))
    if res["tie_rounds"]:
        print(f"({res['tie_rounds']} grammar rounds had several pairs at the maximum; resolved in the reference's map order)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
