"""Scrape throughput and MFU out of training logs into CSV files.

    python extract_metrics.py <input_folder>

Behaviour of the reference's ``extract_metrics.py:8-211``: every ``*.out`` log below the folder is scanned for step
lines (``[rank R] Step: ... | Tokens/s/GPU: 43.1K | ... | MFU: 49.80% | ...``), the first 3 steps are dropped as
warm-up, the rest is averaged and rounded to integers, and the result goes to ``metrics.csv`` beside each log and
to one ``global_metrics.csv`` per sweep directory. Run parameters are parsed from the folder name
(``dp8_tp1_pp1_cp1_mbs4_ga32_sl1024``); ``cp`` is parsed as well (the reference ignores it). Step lines are
accepted with or without torchrun's ``[defaultN]:`` tee prefix.
"""
import argparse
import csv
import glob
import os
import re
from statistics import mean

FIELDS = ["run_name", "status", "dp", "tp", "pp", "cp", "micro_batch_size", "grad_acc", "seq_len", "avg_tokens_s_gpu",
          "avg_mfu"]
WARMUP_STEPS = 3
_MULT = {"T": 1e12, "B": 1e9, "M": 1e6, "K": 1e3}


def parse_folder_name(folder_name):
    def grab(key):
        m = re.search(rf"(?<![a-z]){key}(\d+)", folder_name)
        return int(m.group(1)) if m else None
    return {"dp": grab("dp"), "tp": grab("tp"), "pp": grab("pp"), "cp": grab("cp"), "micro_batch_size": grab("mbs"),
            "grad_acc": grab("ga"), "seq_len": grab("sl")}


def from_readable_format(text):
    if not isinstance(text, str):
        return text
    t = text.strip().upper()
    try:
        return float(t)
    except ValueError:
        pass
    if t[-1] not in _MULT:
        raise ValueError(f"Unknown suffix: {t[-1]}")
    return float(t[:-1]) * _MULT[t[-1]]


def parse_log_line(line):
    tok = re.search(r"Tokens/s/GPU:\s*([\d.]+[KMBT]?)", line)
    mfu = re.search(r"MFU:\s+(\d+\.\d+)%", line)
    return (float(mfu.group(1)) if mfu else None), (from_readable_format(tok.group(1)) if tok else None)


def process_file(filepath):
    toks, mfus = [], []
    with open(filepath, "r", errors="replace") as f:
        for line in f:
            if re.search(r"(\[default\d+\]:)?\[rank \d+\]", line) and "Step:" in line:
                m, t = parse_log_line(line)
                if t is not None:
                    toks.append(t)
                if m is not None:
                    mfus.append(m)
    if len(toks) <= WARMUP_STEPS and len(mfus) <= WARMUP_STEPS:
        print(f"Warning: Not enough data points for {filepath}")
        return None, None
    tok = int(round(mean(toks[WARMUP_STEPS:]))) if len(toks) > WARMUP_STEPS else None
    mfu = int(round(mean(mfus[WARMUP_STEPS:]))) if len(mfus) > WARMUP_STEPS else None
    return mfu, tok


def read_status(status_file):
    try:
        with open(status_file, "r") as f:
            return f.read().strip()
    except OSError:
        return None


def write_csv(row, path):
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=FIELDS)
        w.writeheader()
        w.writerow({k: row.get(k) for k in FIELDS})


def create_subdirectory_metrics(input_folder):
    out_files = glob.glob(os.path.join(input_folder, "**/*.out"), recursive=True)
    print(f"Found {len(out_files)} .out files")
    done = []
    for path in out_files:
        d = os.path.dirname(path)
        row = {"run_name": os.path.basename(d), **parse_folder_name(os.path.basename(d)),
               "status": read_status(os.path.join(d, "status.txt"))}
        mfu, tok = process_file(path)
        row["avg_tokens_s_gpu"], row["avg_mfu"] = tok, mfu
        write_csv(row, os.path.join(d, "metrics.csv"))
        if tok is not None:
            done.append(d)
            print(f"Processed {path} -> metrics.csv")
    return done


def aggregate_metrics(input_folder):
    for top in sorted(glob.glob(os.path.join(input_folder, "*"))):
        if not os.path.isdir(top):
            continue
        rows = []
        for sub in sorted(glob.glob(os.path.join(top, "*"))):
            if not os.path.isdir(sub):
                continue
            name = os.path.basename(sub)
            row = {"run_name": name, "status": read_status(os.path.join(sub, "status.txt")), **parse_folder_name(name),
                   "avg_tokens_s_gpu": -1, "avg_mfu": -1}
            mpath = os.path.join(sub, "metrics.csv")
            if os.path.exists(mpath):
                try:
                    with open(mpath) as f:
                        m = next(csv.DictReader(f))
                    row["avg_tokens_s_gpu"], row["avg_mfu"] = int(m["avg_tokens_s_gpu"]), int(m["avg_mfu"])
                except (StopIteration, ValueError, KeyError, TypeError):
                    pass
            rows.append(row)
        if not rows:
            continue
        with open(os.path.join(top, "global_metrics.csv"), "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=FIELDS)
            w.writeheader()
            w.writerows(rows)
        print(f"Created {os.path.join(top, 'global_metrics.csv')} with {len(rows)} entries")


def main(argv=None):
    p = argparse.ArgumentParser(description="Process log files and create metrics CSVs")
    p.add_argument("input_folder", help="Path to the top-level folder containing experiment subfolders")
    a = p.parse_args(argv)
    print("Creating individual metrics.csv files...")
    create_subdirectory_metrics(a.input_folder)
    print("\nAggregating metrics into global_metrics.csv...")
    aggregate_metrics(a.input_folder)


if __name__ == "__main__":
    main()
