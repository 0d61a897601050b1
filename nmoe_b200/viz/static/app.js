// Dashboard state, the run list, tabs, and the training tab (summary cards + charts with run comparison).
'use strict';

const $ = (id) => document.getElementById(id);

const state = {
  runs: [],              // rows of /api/runs
  primary: null,         // the run whose summary / GPUs / router are shown
  compare: new Set(),    // further runs overlaid on every chart
  tab: 'training',
  tags: ['train/loss', 'optimizer/lr', 'throughput/tokens_per_s_gpu', 'throughput/ms_per_step', 'efficiency/tflops', 'train/grad_norm'],
  colors: new Map(),     // run -> colour, stable while the page lives
  readouts: new Map(),   // canvas -> hover read-out function
};

async function getJSON(url) {
  const r = await fetch(url, { cache: 'no-store' });
  const j = await r.json();
  if (!r.ok) throw new Error(j && j.error ? j.error : r.statusText);
  return j;
}

function colorOf(run) {
  if (!state.colors.has(run)) state.colors.set(run, PALETTE[state.colors.size % PALETTE.length]);
  return state.colors.get(run);
}

function selectedRuns() {
  const out = [];
  if (state.primary) out.push(state.primary);
  for (const r of state.compare) if (r !== state.primary) out.push(r);
  return out;
}

function ago(ts) {
  if (!ts) return 'no metrics';
  const d = Date.now() - ts;
  return d < 0 ? 'now' : fmtDuration(d) + ' ago';
}

// ---------------------------------------------------------------------------------------------- run list
async function loadRuns() {
  const j = await getJSON('/api/runs');
  state.runs = j.runs || [];
  if (!state.primary && state.runs.length) state.primary = state.runs[0].run;
  renderRuns();
}

function renderRuns() {
  const filter = $('run-filter').value.trim().toLowerCase();
  const ul = $('runs');
  ul.innerHTML = '';
  for (const r of state.runs) {
    if (filter && !r.run.toLowerCase().includes(filter)) continue;
    const li = document.createElement('li');
    if (r.run === state.primary) li.className = 'primary';
    const live = r.last_ts && Date.now() - r.last_ts < 120000;
    const status = r.status || (live ? 'running' : '');
    const cb = document.createElement('input');
    cb.type = 'checkbox';
    cb.title = 'overlay this run on the charts';
    cb.checked = state.compare.has(r.run) || r.run === state.primary;
    cb.disabled = r.run === state.primary;
    cb.addEventListener('click', (ev) => {
      ev.stopPropagation();
      if (cb.checked) state.compare.add(r.run); else state.compare.delete(r.run);
      refresh();
    });
    const name = document.createElement('span');
    name.className = 'name';
    name.innerHTML = `<span class="swatch" style="background:${colorOf(r.run)}"></span>${escapeHtml(r.run)}`;
    const dot = document.createElement('span');
    dot.className = 'dot ' + status;
    dot.title = status || 'unknown';
    const meta = document.createElement('span');
    meta.className = 'meta';
    meta.textContent = `step ${r.last_step || 0} · ${ago(r.last_ts)}` + (r.experiment_id ? ` · ${r.experiment_id}` : '');
    li.append(cb, name, dot, meta);
    li.addEventListener('click', () => { state.primary = r.run; state.compare.delete(r.run); renderRuns(); refresh(true); });
    ul.appendChild(li);
  }
}

// ---------------------------------------------------------------------------------------------- charts
function makeChartBox(container, tag, removable) {
  const box = document.createElement('div');
  box.className = 'chart';
  box.dataset.tag = tag;
  const h = document.createElement('h4');
  const title = document.createElement('span');
  title.textContent = tag;
  const tools = document.createElement('span');
  const zoom = document.createElement('a');
  zoom.textContent = 'enlarge';
  zoom.addEventListener('click', () => openChartModal(tag));
  tools.appendChild(zoom);
  if (removable) {
    const rm = document.createElement('a');
    rm.textContent = 'remove';
    rm.addEventListener('click', () => { state.tags = state.tags.filter((t) => t !== tag); box.remove(); });
    tools.appendChild(rm);
  }
  h.append(title, tools);
  const canvas = document.createElement('canvas');
  const legend = document.createElement('div');
  legend.className = 'legend';
  canvas.addEventListener('mousemove', (ev) => {
    const f = state.readouts.get(canvas);
    if (f) legend.innerHTML = f(ev.clientX);
  });
  box.append(h, canvas, legend);
  container.appendChild(box);
  return box;
}

function chartOptions() {
  return { smooth: parseFloat($('smooth').value) || 0, logY: $('logy').checked, xAxis: $('xaxis').value };
}

async function fetchSeries(tag, points) {
  const runs = selectedRuns();
  const got = await Promise.all(runs.map((run) =>
    getJSON(`/api/series?run=${encodeURIComponent(run)}&tag=${encodeURIComponent(tag)}&points=${points}`)
      .then((j) => ({ name: run, color: colorOf(run), points: j.series || [] }))
      .catch(() => ({ name: run, color: colorOf(run), points: [] }))));
  return got;
}

async function drawTagInto(box, tag, points) {
  const canvas = box.querySelector('canvas');
  const series = await fetchSeries(tag, points);
  state.readouts.set(canvas, drawChart(canvas, series, chartOptions()));
  const legend = box.querySelector('.legend');
  if (!legend.innerHTML) {
    legend.innerHTML = series.map((s) => {
      const last = s.points.length ? s.points[s.points.length - 1].value : NaN;
      return `<span class="swatch" style="background:${s.color}"></span>${escapeHtml(s.name)} <b>${fmtNum(last)}</b>`;
    }).join(' &nbsp; ');
  }
}

async function renderCharts(containerId, tags, removable) {
  const container = $(containerId);
  const have = new Map(Array.from(container.children).map((c) => [c.dataset.tag, c]));
  for (const [tag, el] of have) if (!tags.includes(tag)) el.remove();
  await Promise.all(tags.map((tag) => {
    const box = have.get(tag) || makeChartBox(container, tag, removable);
    box.querySelector('.legend').innerHTML = '';
    return drawTagInto(box, tag, 800);
  }));
}

async function openChartModal(tag) {
  const content = $('modal-content');
  content.innerHTML = '';
  const box = makeChartBox(content, tag, false);
  box.querySelector('h4 span:last-child').remove();
  $('modal').hidden = false;
  await drawTagInto(box, tag, 4000);
}

// ---------------------------------------------------------------------------------------------- training tab
const CARD_TAGS = [
  ['train/loss', 'loss', ''],
  ['optimizer/lr', 'learning rate', ''],
  ['throughput/tokens_per_s_gpu', 'tokens / s / GPU', ''],
  ['throughput/ms_per_step', 'ms / step', ''],
  ['efficiency/tflops', 'TFLOP/s / GPU', ''],
  ['train/grad_norm', 'grad norm', ''],
  ['gpu_agg/mean_utilization_gpu', 'GPU utilisation', '%'],
  ['gpu_agg/total_power_w', 'power', 'W'],
  ['eval/CORE', 'CORE (eval)', ''],
  ['router_agg/mean_cv', 'router load CV', ''],
  ['memory/max_alloc_gib', 'peak memory', 'GiB'],
];

function card(key, value, sub) {
  return `<div class="card"><div class="k">${escapeHtml(key)}</div><div class="v">${value}</div><div class="s">${sub || ''}</div></div>`;
}

async function renderTraining(full) {
  if (!state.primary) { $('cards').innerHTML = card('runs', '0', 'no metric files found'); return; }
  const sum = await getJSON(`/api/summary?run=${encodeURIComponent(state.primary)}`).catch(() => ({ summary: {}, steps: {} }));
  const s = sum.summary || {}, steps = sum.steps || {};
  const info = state.runs.find((r) => r.run === state.primary) || {};
  let html = card('run', escapeHtml(state.primary), `step ${info.last_step || 0} · ${info.status || ''} ${ago(info.last_ts)}`);
  for (const [tag, label, unit] of CARD_TAGS) {
    if (tag in s) html += card(label, fmtNum(s[tag]) + (unit ? ' ' + unit : ''), `at step ${steps[tag] !== undefined ? steps[tag] : '?'}`);
  }
  $('cards').innerHTML = html;
  if (full) {
    const tags = await getJSON(`/api/tags?run=${encodeURIComponent(state.primary)}`).catch(() => ({ tags: [] }));
    $('tag-list').innerHTML = (tags.tags || []).map((t) => `<option value="${escapeHtml(t)}">`).join('');
  }
  await renderCharts('charts', state.tags, true);
}

// ---------------------------------------------------------------------------------------------- plumbing
const renderers = { training: renderTraining };      // panels.js adds the other tabs

async function refresh(full) {
  const t0 = performance.now();
  try {
    const f = renderers[state.tab];
    if (f) await f(!!full);
    $('status').textContent = `updated ${new Date().toLocaleTimeString()} (${(performance.now() - t0).toFixed(0)} ms)`;
  } catch (e) {
    $('status').textContent = 'error: ' + e.message;
  }
}

function showTab(name) {
  state.tab = name;
  for (const b of document.querySelectorAll('#tabs button')) b.classList.toggle('on', b.dataset.tab === name);
  for (const s of document.querySelectorAll('.tab')) s.classList.toggle('on', s.id === 'tab-' + name);
  refresh(true);
}

function boot() {
  for (const b of document.querySelectorAll('#tabs button')) b.addEventListener('click', () => showTab(b.dataset.tab));
  $('run-filter').addEventListener('input', renderRuns);
  $('tag-add').addEventListener('click', () => {
    const t = $('tag-input').value.trim();
    if (t && !state.tags.includes(t)) { state.tags.push(t); refresh(); }
    $('tag-input').value = '';
  });
  for (const id of ['smooth', 'logy', 'xaxis']) $(id).addEventListener('change', () => refresh());
  $('modal-close').addEventListener('click', () => { $('modal').hidden = true; });
  $('modal').addEventListener('click', (ev) => { if (ev.target === $('modal')) $('modal').hidden = true; });
  window.addEventListener('resize', () => refresh());
  loadRuns().then(() => refresh(true));
  setInterval(async () => {
    if (!$('auto').checked || document.hidden || !$('modal').hidden) return;
    await loadRuns().catch(() => {});
    if (state.tab !== 'datasets' && state.tab !== 'experiments') refresh();
  }, 5000);
}

document.addEventListener('DOMContentLoaded', boot);
