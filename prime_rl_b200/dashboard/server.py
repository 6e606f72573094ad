"""Run dashboard: a read-only FastAPI app over registered run directories. Per run it serves
the ``metrics.jsonl`` rows (trainer, orchestrator, evals) with a plot, the resolved configs, the
tail of every log file, and a trace browser: the episodes the orchestrator shipped (reward,
advantage, turns) with a token view that colours every sampled token by the engine's
log-probability, the trainer's log-probability, their difference, or the trainer's entropy
(joined from the trainer's annotation stream by trace id)
(reference: src/prime_rl/dashboard/server.py and the ``dashboard`` console script; plain web UI,
no graphics API involved).

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


def _monitor_dir(run_dir: Path) -> Path:
    from ..utils.pathing import get_monitor_dir

    return get_monitor_dir(Path(run_dir))


def read_trace_index(run_dir: Path) -> list[dict]:
    """One summary row per episode (no token arrays), newest last."""
    out = []
    mdir = _monitor_dir(run_dir)
    for f in sorted(mdir.glob("traces_*_*.jsonl")):
        try:
            with open(f) as fh:
                for line_no, line in enumerate(fh):
                    try:
                        t = json.loads(line)
                    except ValueError:
                        continue
                    out.append({"trace_id": t.get("trace_id"), "step": t.get("step"), "env": t.get("env"),
                                "reward": t.get("reward"), "advantage": t.get("advantage"),
                                "turns": len(t.get("turns", [])), "error": t.get("error"),
                                "tokens": sum(len(u.get("completion_ids", [])) for u in t.get("turns", [])),
                                "file": f.name, "line": line_no})
        except OSError:
            continue
    return out


def read_trace(run_dir: Path, trace_id: str) -> dict | None:
    """The full episode plus the trainer's annotations for it (``annotations``: one record per
    branch with per-token ``logprobs`` / ``entropy`` / ``loss_mask``)."""
    mdir = _monitor_dir(run_dir)
    found = None
    for f in sorted(mdir.glob("traces_*_*.jsonl")):
        with open(f) as fh:
            for line in fh:
                if trace_id in line:
                    try:
                        t = json.loads(line)
                    except ValueError:
                        continue
                    if t.get("trace_id") == trace_id:
                        found = t
                        break
        if found:
            break
    if found is None:
        return None
    ann = []
    for f in sorted(mdir.glob("annotations_*.jsonl")):
        with open(f) as fh:
            for line in fh:
                if trace_id in line:
                    try:
                        a = json.loads(line)
                    except ValueError:
                        continue
                    if a.get("trace_id") == trace_id:
                        ann.append(a)
    found["annotations"] = ann
    return found


def read_configs(run_dir: Path) -> dict[str, str]:
    out = {}
    for f in sorted(Path(run_dir).rglob("*.toml"))[:32]:
        try:
            out[str(f.relative_to(run_dir))] = f.read_text()[:200_000]
        except OSError:
            pass
    return out


def read_log_tails(run_dir: Path, lines: int = 200) -> dict[str, str]:
    out = {}
    for f in sorted(Path(run_dir).rglob("*.log"))[:64]:
        try:
            with open(f, "rb") as fh:
                fh.seek(0, 2)
                fh.seek(max(0, fh.tell() - 64 * 1024))
                out[str(f.relative_to(run_dir))] = "\n".join(fh.read().decode(errors="replace").splitlines()[-lines:])
        except OSError:
            pass
    return out


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
</script>
<h2>Traces</h2><button onclick="traces()">refresh</button>
<select id="overlay"><option value="engine">engine logprob</option><option value="trainer">trainer logprob</option>
<option value="diff">trainer - engine</option><option value="entropy">trainer entropy</option></select>
<div style="display:flex;gap:1em"><div id="tl" style="max-height:420px;overflow:auto;min-width:420px;font:12px monospace"></div>
<div id="tv" style="flex:1;font:12px monospace;line-height:1.9"></div></div>
<h2>Episodes</h2>
step <input id="fstep" size="5"> env <input id="fenv" size="10"> reward &ge; <input id="fmin" size="4"> &le; <input id="fmax" size="4">
sort <select id="fsort"><option>step</option><option>reward</option><option>advantage</option><option>tokens</option><option>lag</option></select>
<button onclick="eps(0)">search</button> <button onclick="eps(epOff-50)">&lt;</button> <button onclick="eps(epOff+50)">&gt;</button>
<span id="epinfo"></span><br><canvas id="hist" width="420" height="120"></canvas><canvas id="ser" width="460" height="120"></canvas>
<table id="eptab" style="font:12px monospace;border-collapse:collapse"></table>
<script>
let epOff=0;
function qs(){const p=new URLSearchParams();const v=(id)=>document.getElementById(id).value.trim();
 if(v('fstep'))p.set('step',v('fstep'));if(v('fenv'))p.set('env',v('fenv'));if(v('fmin'))p.set('min_reward',v('fmin'));
 if(v('fmax'))p.set('max_reward',v('fmax'));return p;}
function bars(id,vals,label){const c=document.getElementById(id),g=c.getContext('2d');g.clearRect(0,0,c.width,c.height);
 if(!vals.length)return;const m=Math.max(...vals)||1,w=(c.width-10)/vals.length;vals.forEach((v,i)=>g.fillRect(5+i*w,c.height-14-(c.height-28)*v/m,Math.max(1,w-1),(c.height-28)*v/m));
 g.fillText(label,6,10);}
async function eps(off){epOff=Math.max(0,off);const i=document.getElementById('run').value;const p=qs();p.set('offset',epOff);p.set('limit',50);
 p.set('sort',document.getElementById('fsort').value);const r=await (await fetch(`api/runs/${i}/episodes?`+p)).json();
 document.getElementById('epinfo').textContent=`${r.total} episodes, showing ${r.offset}..${r.offset+r.rows.length}; steps ${r.steps[0]}..${r.steps[1]}; envs ${r.envs.join(', ')}`;
 document.getElementById('eptab').innerHTML='<tr><th>step</th><th>env</th><th>task</th><th>reward</th><th>adv</th><th>tok</th><th>lag</th><th>finish</th><th></th></tr>'+
  r.rows.map(t=>`<tr style="cursor:pointer" onclick="show('${t.trace_id}')"><td>${t.step}</td><td>${t.env}</td><td>${t.task_id}</td><td>${t.reward==null?'-':t.reward.toFixed(3)}</td>`+
  `<td>${t.advantage==null?'-':t.advantage.toFixed(3)}</td><td>${t.tokens}</td><td>${t.lag??'-'}</td><td>${t.finish_reason??''}</td><td>${t.error?'ERR':''}</td></tr>`).join('');
 const h=await (await fetch(`api/runs/${i}/episodes/histogram?`+qs())).json();bars('hist',h.counts||[],`reward histogram, n=${h.n}`);
 const s=await (await fetch(`api/runs/${i}/episodes/series?field=reward`)).json();bars('ser',s.map(x=>x.mean),'mean reward per step');}
</script>
<h2>Configs and logs</h2><button onclick="files()">load</button><pre id="files" style="max-height:400px;overflow:auto;background:#f6f6f6"></pre>
<script>
let cur=null;
async function traces(){const i=document.getElementById('run').value;const r=await (await fetch(`api/runs/${i}/traces`)).json();
 document.getElementById('tl').innerHTML=r.slice(-500).reverse().map(t=>`<div style="cursor:pointer" onclick="show('${t.trace_id}')">`+
 `step ${t.step} ${t.env} r=${(t.reward??0).toFixed(3)} a=${t.advantage==null?'-':t.advantage.toFixed(3)} ${t.tokens} tok${t.error?' ERR':''}</div>`).join('');}
function colour(v,lo,hi){if(v==null)return'#eee';const x=Math.max(0,Math.min(1,(v-lo)/(hi-lo)));return `hsl(${120*x},70%,80%)`;}
async function show(id){const i=document.getElementById('run').value;cur=await (await fetch(`api/runs/${i}/traces/${id}`)).json();render();}
document.getElementById('overlay').onchange=render;
function render(){if(!cur)return;const mode=document.getElementById('overlay').value;const ann=(cur.annotations||[])[0];
 let html=`<b>${cur.env}</b> reward ${cur.reward} advantage ${cur.advantage} policy v${cur.policy_version}<br>`;
 cur.turns.forEach((t,ti)=>{const off=t.prompt_ids.length;html+=`<div><i>turn ${ti}: ${off} prompt tokens, finish ${t.finish_reason}</i><br>`;
  t.completion_ids.forEach((id,k)=>{const e=t.completion_logprobs[k];const tr=ann&&ti===cur.turns.length-1?ann.logprobs[off+k]:null;
   const en=ann&&ti===cur.turns.length-1?ann.entropy[off+k]:null;
   const v=mode==='engine'?e:mode==='trainer'?tr:mode==='diff'?(tr==null?null:tr-e):en;
   const c=mode==='diff'?colour(v==null?null:-Math.abs(v),-1,0):mode==='entropy'?colour(v==null?null:-v,-3,0):colour(v,-5,0);
   html+=`<span title="id ${id} engine ${e} trainer ${tr} entropy ${en}" style="background:${c};padding:1px 3px;margin:1px">${id}</span>`;});
  html+='</div>';});document.getElementById('tv').innerHTML=html;}
async function files(){const i=document.getElementById('run').value;const c=await (await fetch(`api/runs/${i}/configs`)).json();
 const l=await (await fetch(`api/runs/${i}/logs`)).json();
 document.getElementById('files').textContent=Object.entries(c).map(([k,v])=>`### ${k}\n${v}`).join('\n\n')+'\n\n'+
  Object.entries(l).map(([k,v])=>`### ${k}\n${v}`).join('\n\n');}
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

    def run_dir(i: int) -> Path:
        d = dirs()
        if not 0 <= i < len(d):
            raise HTTPException(404, "unknown run")
        return Path(d[i])

    @app.get("/api/runs/{i}/traces")
    def traces(i: int):
        return read_trace_index(run_dir(i))

    @app.get("/api/runs/{i}/traces/{trace_id}")
    def trace(i: int, trace_id: str):
        t = read_trace(run_dir(i), trace_id)
        if t is None:
            raise HTTPException(404, "unknown trace")
        return t

    @app.get("/api/runs/{i}/configs")
    def configs(i: int):
        return read_configs(run_dir(i))

    @app.get("/api/runs/{i}/logs")
    def logs(i: int):
        return read_log_tails(run_dir(i))

    # ------------------------------------------------------------------ episode browser
    indexes: dict[str, "EpisodeIndex"] = {}

    def index_of(i: int):
        from .episodes import EpisodeIndex

        d = run_dir(i)
        idx = indexes.get(str(d))
        if idx is None:
            idx = indexes[str(d)] = EpisodeIndex(_monitor_dir(d))
        return idx.refresh()

    def selected(i, step, min_step, max_step, env, task_id, group_id, min_reward, max_reward, errors, q):
        return index_of(i).select(step=step, min_step=min_step, max_step=max_step, env=env, task_id=task_id,
                                  group_id=group_id, min_reward=min_reward, max_reward=max_reward, errors=errors, text=q)

    @app.get("/api/runs/{i}/episodes")
    def episodes(i: int, step: int | None = None, min_step: int | None = None, max_step: int | None = None,
                 env: str | None = None, task_id: str | None = None, group_id: str | None = None,
                 min_reward: float | None = None, max_reward: float | None = None, errors: bool | None = None,
                 q: str | None = None, sort: str = "step", descending: bool = True, offset: int = 0, limit: int = 100):
        rows = selected(i, step, min_step, max_step, env, task_id, group_id, min_reward, max_reward, errors, q)
        return index_of(i).page(rows, sort=sort, descending=descending, offset=offset, limit=limit)

    @app.get("/api/runs/{i}/episodes/histogram")
    def episodes_histogram(i: int, field: str = "reward", bins: int = 20, step: int | None = None,
                           min_step: int | None = None, max_step: int | None = None, env: str | None = None):
        from .episodes import EpisodeIndex

        return EpisodeIndex.histogram(selected(i, step, min_step, max_step, env, None, None, None, None, None, None),
                                      field, bins)

    @app.get("/api/runs/{i}/episodes/series")
    def episodes_series(i: int, field: str = "reward", env: str | None = None):
        from .episodes import EpisodeIndex

        return EpisodeIndex.series(selected(i, None, None, None, env, None, None, None, None, None, None), field)

    @app.get("/api/runs/{i}/rollouts")
    def rollouts(i: int, step: int | None = None, env: str | None = None, task_id: str | None = None,
                 offset: int = 0, limit: int = 50):
        from .episodes import EpisodeIndex

        groups = EpisodeIndex.rollouts(selected(i, step, None, None, env, task_id, None, None, None, None, None))
        return {"total": len(groups), "groups": groups[offset:offset + max(0, min(limit, 500))]}

    @app.get("/api/runs/{i}/episodes/{trace_id}/timeline")
    def episode_timeline(i: int, trace_id: str):
        from .episodes import timeline

        t = read_trace(run_dir(i), trace_id)
        if t is None:
            raise HTTPException(404, "unknown trace")
        return {"trace_id": trace_id, "reward": t.get("reward"), "advantage": t.get("advantage"), "turns": timeline(t)}

    @app.get("/api/runs/{i}/series")
    def metric_series(i: int, key: str, points: int = 2000, producer: str | None = None):
        from .episodes import downsample

        return downsample(read_metrics(run_dir(i), limit=10 ** 9), key, points, producer)

    @app.get("/api/runs/{i}/logfiles")
    def logfiles(i: int):
        d = run_dir(i)
        out = []
        for f in sorted(d.rglob("*.log"))[:256]:
            try:
                out.append({"name": str(f.relative_to(d)), "size": f.stat().st_size, "mtime": f.stat().st_mtime})
            except OSError:
                pass
        return out

    @app.get("/api/runs/{i}/log")
    def log(i: int, name: str, offset: int | None = None, lines: int = 400):
        from .episodes import read_log

        try:
            return read_log(run_dir(i), name, offset, lines)
        except PermissionError as e:
            raise HTTPException(403, str(e))
        except OSError:
            raise HTTPException(404, "unknown log file")

    @app.get("/api/view/events")
    async def view_events(once: bool = False):
        """Server-sent events: the list of run directories, again whenever a launcher registers a new one."""
        import asyncio

        from fastapi.responses import StreamingResponse

        async def gen():
            last = None
            while True:
                cur = dirs()
                if cur != last:
                    last = cur
                    yield f"event: runs\ndata: {json.dumps(cur)}\n\n"
                    if once:
                        return
                await asyncio.sleep(2.0)

        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/api/view")
    def add_view(body: dict):
        """Registers a run directory with the running dashboard (what launchers call)."""
        path = Path(str(body.get("path", "")))
        if not path.is_dir():
            raise HTTPException(400, "path is not a directory")
        register_output_dir(path)
        return {"runs": dirs()}

    @app.get("/health")
    def health():
        return {"status": "ok"}

    return app
