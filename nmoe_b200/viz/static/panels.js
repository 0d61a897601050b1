// The GPU, router, experiments and datasets tabs.
'use strict';

// ---------------------------------------------------------------------------------------------- GPUs
function bar(frac, warmAt, hotAt) {
  const f = Math.min(1, Math.max(0, frac || 0));
  const cls = f >= hotAt ? 'bar hot' : f >= warmAt ? 'bar warm' : 'bar';
  return `<div class="${cls}"><i style="width:${(f * 100).toFixed(1)}%"></i></div>`;
}

function flag(label, on, bad) {
  return `<span class="flag${on ? ' on' : ''}${on && bad ? ' bad' : ''}">${label}</span>`;
}

async function renderGpu() {
  if (!state.primary) return;
  const j = await getJSON(`/api/gpu?run=${encodeURIComponent(state.primary)}`);
  const agg = j.agg || {};
  $('gpu-agg').innerHTML =
    card('GPUs', String((j.gpus || []).length), '') +
    card('mean utilisation', fmtNum(agg['gpu_agg/mean_utilization_gpu']) + ' %', '') +
    card('memory in use', fmtNum(agg['gpu_agg/total_memory_used_gib']) + ' GiB', 'all GPUs') +
    card('power', fmtNum(agg['gpu_agg/total_power_w']) + ' W', 'all GPUs') +
    card('hottest', fmtNum(agg['gpu_agg/max_temperature_c']) + ' °C', '');
  let html = '';
  for (const g of j.gpus || []) {
    const memFrac = g.memory_total_gib ? g.memory_used_gib / g.memory_total_gib : 0;
    const clkFrac = g.clocks_sm_max_mhz ? g.clocks_sm_mhz / g.clocks_sm_max_mhz : 0;
    html += `<div class="gpu"><h4><span>GPU ${g.index}</span><span class="small">${fmtNum(g.temperature_c)} °C</span></h4>` +
      `<div class="small">utilisation ${fmtNum(g.utilization_gpu)} %</div>${bar((g.utilization_gpu || 0) / 100, 2, 2)}` +
      `<div class="small">memory ${fmtNum(g.memory_used_gib)} / ${fmtNum(g.memory_total_gib)} GiB</div>${bar(memFrac, 0.9, 0.97)}` +
      `<div class="small">power ${fmtNum(g.power_draw_w)} W` + (g.power_limit_w ? ` / ${fmtNum(g.power_limit_w)} W` : '') + `</div>` +
      bar(g.power_limit_w ? g.power_draw_w / g.power_limit_w : (g.power_draw_w || 0) / 1000, 0.9, 0.99) +
      `<div class="small">SM clock ${fmtNum(g.clocks_sm_mhz)}` + (g.clocks_sm_max_mhz ? ` / ${fmtNum(g.clocks_sm_max_mhz)}` : '') + ` MHz</div>` +
      bar(clkFrac, 2, 2) +
      `<div>${flag('power cap', g.throttle_power, false)}${flag('thermal', g.throttle_thermal, true)}` +
      `${flag('hw slowdown', g.throttle_hw_slowdown, true)}${flag('app clocks', g.throttle_apps, false)}` +
      `${flag('ECC ' + (g.ecc_uncorrected || 0), (g.ecc_uncorrected || 0) > 0, true)}</div></div>`;
  }
  $('gpu-grid').innerHTML = html || '<p class="small">this run recorded no GPU telemetry</p>';
  await renderCharts('gpu-charts', ['gpu_agg/mean_utilization_gpu', 'gpu_agg/total_power_w', 'gpu_agg/max_temperature_c',
                                    'gpu_agg/total_memory_used_gib', 'memory/max_alloc_gib'], false);
}

// ---------------------------------------------------------------------------------------------- router
const ROUTER_COLS = [
  // key, label, low end of the colour scale, high end (null = taken from the data)
  ['cv', 'load CV', 0, 1],
  ['entropy', 'entropy', null, null],
  ['max_load', 'max load', null, null],
  ['bias_range', 'bias range', 0, null],
  ['experts_active', 'experts active', null, null],
];

async function renderRouter() {
  if (!state.primary) return;
  const j = await getJSON(`/api/router?run=${encodeURIComponent(state.primary)}`);
  const layers = j.layers || [], agg = j.agg || {};
  $('router-agg').innerHTML = Object.keys(agg).sort().map((k) => card(k.replace('router_agg/', ''), fmtNum(agg[k]), '')).join('') ||
    card('router', '–', 'this run recorded no router statistics');
  if (layers.length) {
    const range = {};
    for (const [key, , lo, hi] of ROUTER_COLS) {
      const vals = layers.map((l) => l[key]).filter(Number.isFinite);
      range[key] = [lo !== null ? lo : Math.min(...vals), hi !== null ? hi : Math.max(...vals)];
    }
    let html = '<table class="heat"><tr><th>layer</th>' + ROUTER_COLS.map((c) => `<th>${c[1]}</th>`).join('') + '</tr>';
    for (const l of layers) {
      html += `<tr><th>${l.idx}</th>`;
      for (const [key] of ROUTER_COLS) {
        const v = l[key];
        // many active experts and high entropy are the healthy end: reverse those scales
        const rev = key === 'entropy' || key === 'experts_active';
        const [lo, hi] = range[key];
        const col = heatColor(rev ? lo + hi - v : v, lo, hi);
        html += `<td style="background:${col}" title="layer ${l.idx} ${key}">${fmtNum(v)}</td>`;
      }
      html += '</tr>';
    }
    $('router-heat').innerHTML = html + '</table>';
  } else {
    $('router-heat').innerHTML = '';
  }
  const tags = Object.keys(agg).sort();
  if (layers.length) {
    const mid = layers[Math.floor(layers.length / 2)].idx;
    const pad = String(mid).padStart(2, '0');
    tags.push(`router/layer_${pad}/cv`, `router/layer_${pad}/max_load`);
  }
  await renderCharts('router-charts', tags, false);
}

// ---------------------------------------------------------------------------------------------- experiments
function table(el, cols, rows, onRow) {
  el.innerHTML = '';
  const head = document.createElement('tr');
  for (const c of cols) {
    const th = document.createElement('th');
    th.textContent = c.label;
    th.addEventListener('click', () => {
      const dir = el.dataset.sort === c.key ? -1 : 1;
      el.dataset.sort = dir === 1 ? c.key : '';
      rows.sort((a, b) => (a[c.key] > b[c.key] ? dir : a[c.key] < b[c.key] ? -dir : 0));
      table(el, cols, rows, onRow);
    });
    head.appendChild(th);
  }
  el.appendChild(head);
  for (const r of rows) {
    const tr = document.createElement('tr');
    tr.className = 'row';
    for (const c of cols) {
      const td = document.createElement('td');
      const v = c.render ? c.render(r) : r[c.key];
      if (c.html) td.innerHTML = v; else td.textContent = v === null || v === undefined ? '' : String(v);
      tr.appendChild(td);
    }
    if (onRow) tr.addEventListener('click', () => onRow(r));
    el.appendChild(tr);
  }
  if (!rows.length) el.insertAdjacentHTML('beforeend', `<tr><td colspan="${cols.length}" class="small">nothing recorded</td></tr>`);
}

function parseJSON(text) {
  try { return text ? JSON.parse(text) : null; } catch (e) { return null; }
}

function showRunDetail(r) {
  const cfg = parseJSON(r.config_json), res = parseJSON(r.results_json);
  $('modal-content').innerHTML =
    `<h3>${escapeHtml(r.run)}</h3>` +
    `<p class="small">${escapeHtml(r.status)} · started ${escapeHtml(r.started_at || '')}` +
    (r.ended_at ? ` · ended ${escapeHtml(r.ended_at)}` : '') +
    ` · git ${escapeHtml((r.git_hash || '').slice(0, 12))}${r.git_dirty ? ' (dirty)' : ''}</p>` +
    `<button id="open-run">open in the training tab</button>` +
    `<h4>results</h4><pre>${escapeHtml(JSON.stringify(res, null, 1) || 'none')}</pre>` +
    `<h4>configuration</h4><pre>${escapeHtml(JSON.stringify(cfg, null, 1) || 'none')}</pre>`;
  $('modal').hidden = false;
  $('open-run').addEventListener('click', () => {
    state.primary = r.run;
    $('modal').hidden = true;
    renderRuns();
    showTab('training');
  });
}

async function showExperimentRuns(exp) {
  const q = exp ? `?experiment_id=${encodeURIComponent(exp.id)}&limit=500` : '?limit=500';
  const j = await getJSON('/api/experiments/runs' + q);
  $('exp-runs-title').textContent = exp ? `runs of ${exp.name || exp.id}` : 'all runs';
  table($('exp-runs'), [
    { key: 'run', label: 'run' },
    { key: 'status', label: 'status', html: true, render: (r) => `<span class="dot ${escapeHtml(r.status)}"></span> ${escapeHtml(r.status)}` },
    { key: 'started_at', label: 'started' },
    { key: 'ended_at', label: 'ended' },
    { key: 'last_step', label: 'last step' },
    { key: 'git_hash', label: 'git', render: (r) => (r.git_hash || '').slice(0, 10) + (r.git_dirty ? '*' : '') },
    { key: 'results_json', label: 'results', render: (r) => {
      const res = parseJSON(r.results_json);
      if (!res) return '';
      return Object.entries(res).filter(([, v]) => typeof v === 'number').slice(0, 4).map(([k, v]) => `${k}=${fmtNum(v)}`).join('  ');
    } },
  ], j.runs || [], showRunDetail);
}

async function renderExperiments() {
  const j = await getJSON('/api/experiments');
  table($('exp-table'), [
    { key: 'name', label: 'experiment', render: (e) => e.name || e.id },
    { key: 'project', label: 'project' },
    { key: 'created_at', label: 'created' },
    { key: 'runs_total', label: 'runs' },
    { key: 'runs_running', label: 'running' },
    { key: 'runs_completed', label: 'completed' },
    { key: 'runs_failed', label: 'failed' },
    { key: 'runs_killed', label: 'killed' },
    { key: 'last_started_at', label: 'last start' },
  ], j.experiments || [], showExperimentRuns);
  await showExperimentRuns(null);
}

// ---------------------------------------------------------------------------------------------- datasets
const ds = { path: '' };

function fmtBytes(n) {
  if (!Number.isFinite(n)) return '';
  const u = ['B', 'KiB', 'MiB', 'GiB', 'TiB'];
  let i = 0;
  while (n >= 1024 && i < u.length - 1) { n /= 1024; i++; }
  return (i ? n.toFixed(1) : String(n)) + ' ' + u[i];
}

function tokensHtml(ids, eos) {
  return (ids || []).map((t) => `<span class="tok${t === eos ? ' eos' : ''}">${t}</span>`).join('');
}

async function dsOpenDir(path) {
  ds.path = path;
  const j = await getJSON('/api/datasets?path=' + encodeURIComponent(path));
  const parts = path.split('/').filter(Boolean);
  const crumbs = ['<a data-p="">root</a>'];
  parts.forEach((p, i) => crumbs.push(`<a data-p="${escapeHtml(parts.slice(0, i + 1).join('/'))}">${escapeHtml(p)}</a>`));
  $('ds-crumbs').innerHTML = crumbs.join(' / ');
  for (const a of $('ds-crumbs').querySelectorAll('a')) {
    a.style.cursor = 'pointer';
    a.addEventListener('click', () => dsOpenDir(a.dataset.p));
  }
  const rows = (j.entries || []).slice().sort((a, b) => (a.kind === b.kind ? (a.name < b.name ? -1 : 1) : a.kind === 'dir' ? -1 : 1));
  table($('ds-entries'), [
    { key: 'name', label: 'name', render: (e) => (e.kind === 'dir' ? e.name + '/' : e.name) },
    { key: 'size', label: 'size', render: (e) => (e.kind === 'dir' ? '' : fmtBytes(e.size)) },
    { key: 'mtime_ms', label: 'modified', render: (e) => (e.mtime_ms ? new Date(e.mtime_ms).toLocaleString() : '') },
  ], rows, (e) => {
    const p = (path ? path + '/' : '') + e.name;
    if (e.kind === 'dir') dsOpenDir(p); else dsOpenFile(p);
  });
  // a directory with a manifest is a prepared dataset; one with such sub-directories is a flow output
  if (rows.some((e) => e.name === 'manifest.json')) {
    const m = await getJSON('/api/datasets/manifest?path=' + encodeURIComponent(path) + '&limit_shards=20').catch(() => null);
    if (m) $('ds-detail').innerHTML = `<h4>dataset manifest</h4><pre>${escapeHtml(JSON.stringify(m, null, 1))}</pre>`;
  } else if (rows.some((e) => e.kind === 'dir')) {
    const f = await getJSON('/api/datasets/pipeline?path=' + encodeURIComponent(path)).catch(() => null);
    if (f && f.sources && f.sources.length) $('ds-detail').innerHTML = `<h4>prepared sources under this directory</h4><pre>${escapeHtml(JSON.stringify(f, null, 1))}</pre>`;
  }
}

async function dsOpenFile(path) {
  const q = encodeURIComponent(path);
  const meta = await getJSON('/api/datasets/meta?path=' + q).catch((e) => ({ error: e.message }));
  let html = `<h4>${escapeHtml(path)}</h4><pre>${escapeHtml(JSON.stringify(meta, null, 1))}</pre>`;
  if (meta.kind === 'token_shard') {
    const st = await getJSON('/api/datasets/shard/stats?path=' + q).catch(() => null);
    if (st) html += `<h4>token statistics</h4><pre>${escapeHtml(JSON.stringify(st, null, 1))}</pre>`;
    html += `<h4>tokens <input id="ds-off" type="number" value="0" min="0" size="10"> <button id="ds-win">show 256 from here</button></h4><div id="ds-tokens"></div>`;
    const idx = path.replace(/\.npy$/, '.idx');
    html += `<h4>document <input id="ds-doc" type="number" value="0" min="0" size="8"> <button id="ds-docbtn">show</button></h4><div id="ds-docout"></div>`;
    $('ds-detail').innerHTML = html;
    const win = async () => {
      const w = await getJSON(`/api/datasets/shard/window?path=${q}&offset=${parseInt($('ds-off').value, 10) || 0}&length=256`);
      $('ds-tokens').innerHTML = tokensHtml(w.ids, st ? st.eos_token_id : undefined) + (w.text ? `<pre>${escapeHtml(w.text)}</pre>` : '');
    };
    $('ds-win').addEventListener('click', win);
    $('ds-docbtn').addEventListener('click', async () => {
      const d = await getJSON(`/api/datasets/index/doc?path=${encodeURIComponent(idx)}&doc_idx=${parseInt($('ds-doc').value, 10) || 0}&max_tokens=2048`)
        .catch((e) => ({ error: e.message }));
      $('ds-docout').innerHTML = d.error ? `<p class="small">${escapeHtml(d.error)}</p>` :
        `<p class="small">tokens [${d.start}, ${d.end}) · ${d.tokens} tokens</p>` + tokensHtml(d.ids) + (d.text ? `<pre>${escapeHtml(d.text)}</pre>` : '');
    });
    win().catch(() => {});
    return;
  }
  if (meta.kind === 'index') {
    const h = await getJSON('/api/datasets/index/header?path=' + q).catch(() => null);
    if (h) html += `<h4>index</h4><pre>${escapeHtml(JSON.stringify(h, null, 1))}</pre>`;
  } else {
    const pv = await getJSON('/api/datasets/preview?path=' + q + '&max_bytes=65536').catch(() => null);
    if (pv) html += `<h4>preview (${fmtBytes(pv.bytes)})</h4><pre>${escapeHtml(pv.text !== undefined ? pv.text : pv.hex)}</pre>`;
  }
  $('ds-detail').innerHTML = html;
}

async function renderDatasets(full) {
  if (full || !$('ds-entries').children.length) await dsOpenDir(ds.path);
}

renderers.gpu = renderGpu;
renderers.router = renderRouter;
renderers.experiments = renderExperiments;
renderers.datasets = renderDatasets;
