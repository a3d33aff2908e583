"""Send a checkpoint to the evaluation service: convert -> archive -> resumable upload -> job -> wait.

    python scripts/submit_eval.py <dcp checkpoint dir | HF model dir> --name my-model
           [--family llama|gemma|deepseek|glm4] [--model-name X --flavor Y] [--tokenizer T]
           [--tasks task1,task2] [--api-url URL] [--token TOKEN] [--compression zstd|gz|none]
           [--no-wait] [--keep-archive]

The service speaks the tus resumable-upload protocol (``POST /api/tus/`` creates an upload of
``Upload-Length`` bytes, ``PATCH /api/tus/<id>`` appends a chunk at ``Upload-Offset``, ``HEAD`` reports
the offset), then ``POST /api/uploads/<id>/finalize``, ``POST /api/jobs`` and ``GET /api/jobs/<id>``
(reference: scripts/submit_eval.py:202-563).  An interrupted upload resumes from the server's offset:
its id is remembered in ``<archive>.upload.json``.  ``EVAL_API_URL`` / ``EVAL_TOKEN`` may come from
the environment or a ``.env`` file at the repository root.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tarfile
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

CHUNK = 5 * 1024 * 1024
TERMINAL = {"COMPLETED", "FAILED", "CANCELLED", "ERROR"}


def load_dotenv(path: Path = ROOT / ".env") -> None:
    if not path.is_file():
        return
    for line in path.read_text().splitlines():
        line = line.strip()
        if line and not line.startswith("#") and "=" in line:
            k, v = line.split("=", 1)
            if k.strip() in ("EVAL_API_URL", "EVAL_TOKEN"):
                os.environ.setdefault(k.strip(), v.strip().strip("\"'"))


def is_hf_dir(p: Path) -> bool:
    return (p / "config.json").is_file() and any(p.glob("*.safetensors"))


def ensure_hf_dir(src: Path, work: Path, family: str | None, model_name: str | None, flavor: str | None,
                  tokenizer: str | None) -> Path:
    """An HF directory for ``src``: itself if it already is one, else a conversion of the DCP checkpoint."""
    if is_hf_dir(src):
        return src
    from maester_b200.convert.cli import convert_from_dcp
    from maester_b200.convert.io import find_job_config

    job = find_job_config(src) or {}
    model_name = model_name or job.get("model_name")
    family = family or model_name
    if not family:
        raise SystemExit("cannot tell the model family: pass --family (or --model-name/--flavor)")
    out = work / "hf"
    convert_from_dcp(family, str(src), str(out), model_name=model_name, flavor=flavor or job.get("flavor"),
                     tokenizer=tokenizer or job.get("tokenizer_name"),
                     chat_template="chatml" if job.get("sft") else None)
    return out


def make_archive(src: Path, dst_stem: Path, compression: str = "zstd") -> Path:
    """tar of ``src`` compressed with zstd (CLI, multi-threaded) when available, else gzip / none."""
    if compression == "zstd" and shutil.which("zstd") is None:
        compression = "gz"
    if compression == "zstd":
        out = dst_stem.with_suffix(".tar.zst")
        tar = subprocess.Popen(["tar", "-C", str(src.parent), "-cf", "-", src.name], stdout=subprocess.PIPE)
        with open(out, "wb") as f:
            z = subprocess.run(["zstd", "-T0", "-3", "-q", "-c"], stdin=tar.stdout, stdout=f)
        if tar.wait() != 0 or z.returncode != 0:
            raise RuntimeError("tar | zstd failed")
        return out
    mode, suffix = ("w:gz", ".tar.gz") if compression == "gz" else ("w", ".tar")
    out = dst_stem.with_suffix(suffix)
    with tarfile.open(out, mode) as t:
        t.add(src, arcname=src.name)
    return out


class EvalClient:
    def __init__(self, api_url: str, token: str | None, session=None):
        import requests
        from requests.adapters import HTTPAdapter
        from urllib3.util.retry import Retry

        self.api = api_url.rstrip("/")
        self.s = session or requests.Session()
        adapter = HTTPAdapter(max_retries=Retry(total=3, backoff_factor=0.3, status_forcelist=[500, 502, 503, 504]))
        self.s.mount("http://", adapter)
        self.s.mount("https://", adapter)
        self.h = {"Authorization": f"Bearer {token}"} if token else {}

    # ---- tus upload
    def _offset(self, upload_id: str) -> int | None:
        r = self.s.head(f"{self.api}/api/tus/{upload_id}", headers={**self.h, "Tus-Resumable": "1.0.0"})
        return int(r.headers.get("Upload-Offset", "0")) if r.status_code == 200 else None

    def upload(self, archive: Path, name: str, progress=lambda done, total: None) -> str:
        size = archive.stat().st_size
        memo = Path(str(archive) + ".upload.json")
        upload_id, offset = None, 0
        if memo.is_file():
            d = json.loads(memo.read_text())
            if d.get("file_size") == size and d.get("api_url") == self.api:
                off = self._offset(d["upload_id"])
                if off is not None:
                    upload_id, offset = d["upload_id"], off
        if upload_id is None:
            import base64
            meta = ",".join(f"{k} {base64.b64encode(v.encode()).decode()}" for k, v in
                            {"filename": archive.name, "name": name}.items())
            r = self.s.post(f"{self.api}/api/tus/", headers={**self.h, "Tus-Resumable": "1.0.0",
                                                             "Upload-Length": str(size), "Upload-Metadata": meta})
            r.raise_for_status()
            upload_id = r.headers["Location"].rstrip("/").rsplit("/", 1)[-1]
            memo.write_text(json.dumps({"upload_id": upload_id, "file_size": size, "api_url": self.api}))
        with open(archive, "rb") as f:
            while offset < size:
                f.seek(offset)
                chunk = f.read(CHUNK)
                r = self.s.patch(f"{self.api}/api/tus/{upload_id}", data=chunk,
                                 headers={**self.h, "Tus-Resumable": "1.0.0", "Upload-Offset": str(offset),
                                          "Content-Type": "application/offset+octet-stream"})
                if r.status_code in (200, 204):
                    offset = int(r.headers.get("Upload-Offset", offset + len(chunk)))
                else:  # offset mismatch or transient error: ask the server where it is
                    off = self._offset(upload_id)
                    if off is None:
                        r.raise_for_status()
                        raise RuntimeError(f"upload {upload_id} lost")
                    offset = off
                    time.sleep(0.5)
                progress(offset, size)
        r = self.s.post(f"{self.api}/api/uploads/{upload_id}/finalize", headers=self.h, json={"name": name})
        r.raise_for_status()
        memo.unlink(missing_ok=True)
        return r.json().get("model_id", upload_id)

    # ---- jobs
    def submit(self, model_id: str, name: str, tasks: list[str] | None, extra: dict | None = None) -> str:
        body = {"model_id": model_id, "name": name}
        if tasks:
            body["tasks"] = tasks
        body.update(extra or {})
        r = self.s.post(f"{self.api}/api/jobs", headers=self.h, json=body)
        r.raise_for_status()
        return str(r.json()["job_id"] if "job_id" in r.json() else r.json()["id"])

    def job(self, job_id: str) -> dict:
        r = self.s.get(f"{self.api}/api/jobs/{job_id}", headers=self.h)
        r.raise_for_status()
        return r.json()

    def wait(self, job_id: str, poll_s: float = 10.0, timeout_s: float = 24 * 3600, out=print) -> dict:
        t0, last = time.time(), None
        while True:
            j = self.job(job_id)
            status = str(j.get("status", "UNKNOWN")).upper()
            if status != last:
                out(f"[{time.strftime('%H:%M:%S')}] job {job_id}: {status}")
                last = status
            if status in TERMINAL or time.time() - t0 > timeout_s:
                return j
            time.sleep(poll_s)


def print_results(job: dict) -> None:
    for ev in job.get("evaluations", job.get("results", [])) or []:
        metrics = ev.get("metrics", {})
        if "error" in metrics:
            print(f"  {ev.get('task', '?')}: ERROR {metrics['error']}")
        else:
            shown = ", ".join(f"{k}={v:.4f}" if isinstance(v, float) else f"{k}={v}" for k, v in metrics.items())
            print(f"  {ev.get('task', '?')}: {shown}")


def main(argv=None) -> int:
    load_dotenv()
    ap = argparse.ArgumentParser(description="Submit a model to the evaluation service")
    ap.add_argument("model_path")
    ap.add_argument("--name", required=True)
    ap.add_argument("--family")
    ap.add_argument("--model-name")
    ap.add_argument("--flavor")
    ap.add_argument("--tokenizer")
    ap.add_argument("--tasks", default="")
    ap.add_argument("--api-url", default=os.environ.get("EVAL_API_URL", "http://localhost:8080"))
    ap.add_argument("--token", default=None)
    ap.add_argument("--compression", choices=["zstd", "gz", "none"], default="zstd")
    ap.add_argument("--no-wait", action="store_true")
    ap.add_argument("--keep-archive", action="store_true")
    a = ap.parse_args(argv)
    token = a.token or os.environ.get("EVAL_TOKEN") or os.environ.get("USER_TOKEN")
    work = Path(tempfile.mkdtemp(prefix="submit_eval_"))
    try:
        hf_dir = ensure_hf_dir(Path(a.model_path), work, a.family, a.model_name, a.flavor, a.tokenizer)
        print(f"archiving {hf_dir} ...")
        archive = make_archive(hf_dir, work / a.name, a.compression)
        print(f"archive {archive.name}: {archive.stat().st_size / 2**20:.1f} MiB")
        client = EvalClient(a.api_url, token)
        model_id = client.upload(archive, a.name, lambda d, t: print(f"\ruploaded {100 * d / t:5.1f}%", end="", flush=True))
        print(f"\nmodel id {model_id}")
        job_id = client.submit(model_id, a.name, [t for t in a.tasks.split(",") if t])
        print(f"job {job_id}: {a.api_url}/api/jobs/{job_id}")
        if a.no_wait:
            return 0
        job = client.wait(job_id)
        print_results(job)
        return 0 if str(job.get("status", "")).upper() == "COMPLETED" else 1
    finally:
        if not a.keep_archive:
            shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
