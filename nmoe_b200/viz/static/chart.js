// Line charts on a 2-D canvas: several series per chart, linear or log y, step or wall-time x, exponential smoothing,
// a hover read-out.  No dependencies.
'use strict';

const PALETTE = ['#6ea8fe', '#f5b14c', '#4cc38a', '#f2555a', '#b48efa', '#5ad1e6', '#f78fb3', '#c3d15a'];

function fmtNum(v) {
  if (v === null || v === undefined || Number.isNaN(v)) return '–';
  const a = Math.abs(v);
  if (a === 0) return '0';
  if (a >= 1e9) return (v / 1e9).toFixed(2) + 'G';
  if (a >= 1e6) return (v / 1e6).toFixed(2) + 'M';
  if (a >= 1e4) return (v / 1e3).toFixed(1) + 'k';
  if (a >= 100) return v.toFixed(0);
  if (a >= 1) return v.toFixed(3);
  if (a >= 1e-3) return v.toFixed(4);
  return v.toExponential(2);
}

function fmtDuration(ms) {
  const s = Math.max(0, ms / 1000);
  if (s < 90) return s.toFixed(0) + 's';
  if (s < 5400) return (s / 60).toFixed(1) + 'm';
  return (s / 3600).toFixed(2) + 'h';
}

// exponential moving average with bias correction, so the first points are not dragged toward zero
function smoothSeries(ys, alpha) {
  if (!(alpha > 0)) return ys;
  const out = new Array(ys.length);
  let acc = 0, norm = 0;
  for (let i = 0; i < ys.length; i++) {
    acc = alpha * acc + (1 - alpha) * ys[i];
    norm = alpha * norm + (1 - alpha);
    out[i] = acc / norm;
  }
  return out;
}

function niceTicks(lo, hi, n) {
  if (!(hi > lo)) return [lo];
  const raw = (hi - lo) / Math.max(1, n);
  const mag = Math.pow(10, Math.floor(Math.log10(raw)));
  const norm = raw / mag;
  const step = (norm < 1.5 ? 1 : norm < 3 ? 2 : norm < 7 ? 5 : 10) * mag;
  const out = [];
  for (let v = Math.ceil(lo / step) * step; v <= hi + step * 1e-9; v += step) out.push(v);
  return out;
}

// series: [{name, color, points: [{step, ts_ms, value}]}];  opts: {logY, smooth, xAxis: 'step' | 'time'}
// Returns a function (clientX) -> read-out text for the nearest x, used by the hover handler.
function drawChart(canvas, series, opts) {
  const dpr = window.devicePixelRatio || 1;
  const W = canvas.clientWidth, H = canvas.clientHeight;
  canvas.width = Math.round(W * dpr);
  canvas.height = Math.round(H * dpr);
  const g = canvas.getContext('2d');
  g.setTransform(dpr, 0, 0, dpr, 0, 0);
  g.clearRect(0, 0, W, H);
  const css = getComputedStyle(document.documentElement);
  const cLine = css.getPropertyValue('--line').trim() || '#333';
  const cDim = css.getPropertyValue('--dim').trim() || '#888';
  const m = { l: 52, r: 10, t: 8, b: 22 };
  const useTime = opts.xAxis === 'time';
  const logY = !!opts.logY;

  const prepared = series.map((s) => {
    const pts = s.points.filter((p) => Number.isFinite(p.value) && (!logY || p.value > 0));
    const t0 = pts.length ? pts[0].ts_ms : 0;
    const xs = pts.map((p) => (useTime ? p.ts_ms - t0 : p.step));
    const raw = pts.map((p) => p.value);
    const ys = smoothSeries(raw, opts.smooth || 0);
    return { name: s.name, color: s.color, xs, ys, raw };
  }).filter((s) => s.xs.length > 0);

  g.font = '11px system-ui, sans-serif';
  if (!prepared.length) {
    g.fillStyle = cDim;
    g.fillText('no data', m.l, H / 2);
    return () => '';
  }
  let x0 = Infinity, x1 = -Infinity, y0 = Infinity, y1 = -Infinity;
  for (const s of prepared) {
    for (let i = 0; i < s.xs.length; i++) {
      const y = logY ? Math.log10(s.ys[i]) : s.ys[i];
      if (s.xs[i] < x0) x0 = s.xs[i];
      if (s.xs[i] > x1) x1 = s.xs[i];
      if (y < y0) y0 = y;
      if (y > y1) y1 = y;
    }
  }
  if (x1 === x0) x1 = x0 + 1;
  if (y1 === y0) { y1 = y0 + (Math.abs(y0) || 1) * 0.05; y0 = y0 - (Math.abs(y0) || 1) * 0.05; }
  const pad = (y1 - y0) * 0.05;
  y0 -= pad; y1 += pad;
  const X = (x) => m.l + (x - x0) / (x1 - x0) * (W - m.l - m.r);
  const Y = (y) => H - m.b - ((logY ? Math.log10(y) : y) - y0) / (y1 - y0) * (H - m.t - m.b);

  // grid and labels
  g.strokeStyle = cLine; g.fillStyle = cDim; g.lineWidth = 1;
  for (const t of niceTicks(y0, y1, 5)) {
    const py = H - m.b - (t - y0) / (y1 - y0) * (H - m.t - m.b);
    g.beginPath(); g.moveTo(m.l, py); g.lineTo(W - m.r, py); g.stroke();
    g.textAlign = 'right';
    g.fillText(fmtNum(logY ? Math.pow(10, t) : t), m.l - 4, py + 3);
  }
  for (const t of niceTicks(x0, x1, 6)) {
    const px = X(t);
    g.beginPath(); g.moveTo(px, H - m.b); g.lineTo(px, H - m.b + 3); g.stroke();
    g.textAlign = 'center';
    g.fillText(useTime ? fmtDuration(t) : fmtNum(t), px, H - 6);
  }

  // the raw series faintly under the smoothed one
  for (const s of prepared) {
    if (opts.smooth > 0) {
      g.globalAlpha = 0.25; g.strokeStyle = s.color; g.beginPath();
      for (let i = 0; i < s.xs.length; i++) { const px = X(s.xs[i]), py = Y(s.raw[i]); if (i) g.lineTo(px, py); else g.moveTo(px, py); }
      g.stroke(); g.globalAlpha = 1;
    }
    g.strokeStyle = s.color; g.lineWidth = 1.5; g.beginPath();
    for (let i = 0; i < s.xs.length; i++) { const px = X(s.xs[i]), py = Y(s.ys[i]); if (i) g.lineTo(px, py); else g.moveTo(px, py); }
    g.stroke(); g.lineWidth = 1;
    if (s.xs.length === 1) { g.fillStyle = s.color; g.fillRect(X(s.xs[0]) - 2, Y(s.ys[0]) - 2, 4, 4); g.fillStyle = cDim; }
  }

  return function readout(clientX) {
    const rect = canvas.getBoundingClientRect();
    const x = x0 + (clientX - rect.left - m.l) / (W - m.l - m.r) * (x1 - x0);
    const parts = [];
    for (const s of prepared) {
      // nearest sample by binary search on the sorted x values
      let lo = 0, hi = s.xs.length - 1;
      while (hi - lo > 1) { const mid = (lo + hi) >> 1; if (s.xs[mid] < x) lo = mid; else hi = mid; }
      const i = Math.abs(s.xs[lo] - x) <= Math.abs(s.xs[hi] - x) ? lo : hi;
      parts.push(`<span class="swatch" style="background:${s.color}"></span>${escapeHtml(s.name)} ` +
                 `${useTime ? fmtDuration(s.xs[i]) : 'step ' + s.xs[i]}: <b>${fmtNum(s.ys[i])}</b>`);
    }
    return parts.join(' &nbsp; ');
  };
}

function escapeHtml(s) {
  return String(s).replace(/[&<>"']/g, (c) => ({ '&': '&amp;', '<': '&lt;', '>': '&gt;', '"': '&quot;', "'": '&#39;' }[c]));
}

// value -> colour on a blue -> yellow -> red scale; lo and hi are the ends of the scale
function heatColor(v, lo, hi) {
  if (!Number.isFinite(v)) return '#333';
  const t = Math.min(1, Math.max(0, (v - lo) / ((hi - lo) || 1)));
  const h = 220 - 220 * t;
  return `hsl(${h.toFixed(0)}, 60%, ${(30 + 10 * t).toFixed(0)}%)`;
}
