"""Run dashboard: a small FastAPI app that lists registered run directories and serves their
``metrics.jsonl`` rows (trainer, orchestrator, evals) as JSON plus a single-page plot
(reference: the ``dashboard`` console script, src/prime_rl/entrypoints/dashboard.py; plain web
UI, no graphics API involved).

Registry: ``~/.cache/prime-rl-b200/dashboard/dirs.json`` (launchers add their output
directory; the list is re-read on every request, so new runs appear without a restart).
"""

from __future__ import annotations

import fcntl
import json
import os
from contextlib import contextmanager
from pathlib import Path

STATE_DIR = Path(os.environ.get("PRL_DASHBOARD_STATE", Path.home() / ".cache" / "prime-rl-b200" / "dashboard"))
DIRS_FILE = STATE_DIR / "dirs.json"


@contextmanager
def registry_lock():
    STATE_DIR.mkdir(parents=True, exist_ok=True)
    with open(STATE_DIR / ".lock", "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        yield


def registered_dirs() -> list[str]:
    try:
        return list(json.loads(DIRS_FILE.read_text()))
    except (OSError, ValueError):
        return []


def register_output_dir(path: Path) -> None:
    """Idempotent, atomic (write to a temporary file, then rename)."""
    with registry_lock():
        dirs = registered_dirs()
        entry = str(Path(path).resolve())
        if entry in dirs:
            return
        dirs.append(entry)
        tmp = DIRS_FILE.with_suffix(".tmp")
        tmp.write_text(json.dumps(dirs))
        tmp.replace(DIRS_FILE)


def read_metrics(run_dir: Path, limit: int = 20000) -> list[dict]:
    rows = []
    for f in sorted(Path(run_dir).rglob("metrics.jsonl")) + sorted(Path(run_dir).rglob("evals.jsonl")):
        try:
            with open(f) as fh:
                for line in fh:
                    line = line.strip()
                    if line:
                        try:
                            rows.append(json.loads(line))
                        except ValueError:
                            pass      # a row that is still being written
        except OSError:
            continue
    return rows[-limit:]


_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>prime-rl-b200 runs</title>
<style>body{font-family:sans-serif;margin:1.5em}canvas{border:1px solid #ccc;margin:.4em}select{margin:.3em}</style></head>
<body><h2>Runs</h2><select id="run"></select><select id="key"></select><br><canvas id="c" width="900" height="360"></canvas>
<script>
let rows=[];
async function runs(){const r=await (await fetch('api/runs')).json();const s=document.getElementById('run');
 s.innerHTML=r.map((d,i)=>`<option value="${i}">${d}</option>`).join('');s.onchange=load;if(r.length)load();}
async function load(){const i=document.getElementById('run').value;rows=await (await fetch(`api/runs/${i}/metrics`)).json();
 const keys=[...new Set(rows.flatMap(r=>Object.keys(r).filter(k=>typeof r[k]==='number'&&k!=='step')))].sort();
 const k=document.getElementById('key');k.innerHTML=keys.map(x=>`<option>${x}</option>`).join('');k.onchange=draw;draw();}
function draw(){const k=document.getElementById('key').value;const pts=rows.filter(r=>typeof r[k]==='number'&&typeof r.step==='number');
 const c=document.getElementById('c'),g=c.getContext('2d');g.clearRect(0,0,c.width,c.height);if(!pts.length)return;
 const xs=pts.map(p=>p.step),ys=pts.map(p=>p[k]);const x0=Math.min(...xs),x1=Math.max(...xs)||1,y0=Math.min(...ys),y1=Math.max(...ys);
 g.beginPath();pts.forEach((p,i)=>{const x=20+(c.width-40)*(p.step-x0)/((x1-x0)||1),y=c.height-20-(c.height-40)*(p[k]-y0)/((y1-y0)||1);
 i?g.lineTo(x,y):g.moveTo(x,y);});g.stroke();g.fillText(`${k}: ${y0.toPrecision(4)} .. ${y1.toPrecision(4)}  steps ${x0}..${x1}`,24,14);}
runs();setInterval(load,10000);
</script></body></html>"""


def build_app(extra_dirs: list[str] | None = None):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import HTMLResponse

    app = FastAPI(title="prime-rl-b200 dashboard")

    def dirs() -> list[str]:
        seen, out = set(), []
        for d in (extra_dirs or []) + registered_dirs():
            if d not in seen:
                seen.add(d)
                out.append(d)
        return out

    @app.get("/", response_class=HTMLResponse)
    def index():
        return _PAGE

    @app.get("/api/runs")
    def runs():
        return dirs()

    @app.get("/api/runs/{i}/metrics")
    def metrics(i: int):
        d = dirs()
        if not 0 <= i < len(d):
            raise HTTPException(404, "unknown run")
        return read_metrics(Path(d[i]))

    @app.get("/health")
    def health():
        return {"status": "ok"}

    return app
