// Triune Studio front-end: one page, no build step, no dependencies. Talks to the server's /v1 API and /ws/telemetry.
"use strict";
const $ = (s, r = document) => r.querySelector(s);
const $$ = (s, r = document) => Array.from(r.querySelectorAll(s));
const el = (tag, attrs = {}, ...kids) => {
  const e = document.createElement(tag);
  for (const [k, v] of Object.entries(attrs)) { if (k === "class") e.className = v; else if (k.startsWith("on")) e.addEventListener(k.slice(2), v); else e.setAttribute(k, v); }
  for (const k of kids) e.append(k);
  return e;
};
async function api(path, body, method) {
  const opt = body === undefined ? { method: method || "GET" } : { method: method || "POST", headers: { "Content-Type": "application/json" }, body: JSON.stringify(body) };
  const r = await fetch(path, opt);
  const text = await r.text();
  let data; try { data = text ? JSON.parse(text) : {}; } catch (e) { data = { detail: text }; }
  if (!r.ok) throw new Error(data.detail || r.statusText);
  return data;
}
const fmt = (x, d = 3) => (typeof x === "number" ? (Math.abs(x) >= 1000 ? x.toFixed(0) : x.toPrecision(d)) : String(x));
const say = (node, text, bad) => { node.textContent = text; node.style.color = bad ? "var(--bad)" : ""; };

// ---------------------------------------------------------------- tabs
$$("#tabs button").forEach(b => b.onclick = () => {
  $$("#tabs button").forEach(x => x.classList.toggle("on", x === b));
  $$(".tab").forEach(t => t.classList.toggle("on", t.id === "tab-" + b.dataset.tab));
  if (b.dataset.tab === "system") refreshSystem();
  if (b.dataset.tab === "train") refreshCheckpoints();
  if (b.dataset.tab === "tune") refreshAdapters();
  if (b.dataset.tab === "graph") { loadCatalog(); drawWires(); }
});

// ---------------------------------------------------------------- models
async function refreshModels() {
  try {
    const m = await api("/v1/models");
    const sel = $("#model-select"); sel.innerHTML = "";
    for (const d of m.data) sel.append(el("option", { value: d.id }, d.params ? `${d.id} (${d.params})` : d.id));
    const a = await api("/v1/models/active");
    showActive(a.loaded ? a : null);
  } catch (e) { say($("#model-active"), e.message, true); }
}
function showActive(a) {
  $("#model-active").textContent = a ? `${a.model_id} · ${fmt(a.params / 1e6)}M · ${a.precision}` : "no model";
  $("#model-active").classList.toggle("on", !!a);
}
$("#model-load").onclick = async () => {
  say($("#model-active"), "loading…");
  try { showActive(await api("/v1/models/load", { model: $("#model-select").value, precision: $("#precision-select").value || null })); session = null; }
  catch (e) { say($("#model-active"), e.message, true); }
};

// ---------------------------------------------------------------- telemetry socket
let lossSeries = [];
function connectTelemetry() {
  const ws = new WebSocket((location.protocol === "https:" ? "wss://" : "ws://") + location.host + "/ws/telemetry");
  ws.onopen = () => { $("#link").textContent = "live"; $("#link").className = "pill on"; };
  ws.onclose = () => { $("#link").textContent = "offline"; $("#link").className = "pill off"; setTimeout(connectTelemetry, 2000); };
  ws.onmessage = ev => {
    const m = JSON.parse(ev.data);
    if (m.type === "hello" && m.model) showActive(m.model);
    if (m.type === "train") { lossSeries.push([m.step, m.loss]); if (lossSeries.length > 2000) lossSeries.shift(); drawLoss(); showTrain(m); }
    if ((m.type === "heartbeat" || m.type === "hello") && m.training) showTrain(m.training);
    if (m.type === "finetune") say($("#ft-status"), `step ${m.step}  loss ${fmt(m.loss)}`);
    if (m.type === "dag_event") onDagEvent(m.data);
  };
}

// ---------------------------------------------------------------- chat
let session = null, activeRequest = null;
function addMsg(who, text, cls) {
  const body = el("div", {}, text);
  const m = el("div", { class: "msg " + (cls || "") }, el("div", { class: "who" }, who), body);
  $("#chat-log").append(m); $("#chat-log").scrollTop = 1e9;
  return body;
}
$("#chat-input").addEventListener("keydown", e => { if (e.key === "Enter" && !e.shiftKey) { e.preventDefault(); $("#chat-form").requestSubmit(); } });
$("#chat-reset").onclick = async () => { if (session) { try { await api("/v1/chat/sessions/" + session, undefined, "DELETE"); } catch (e) { /* gone already */ } } session = null; $("#chat-log").innerHTML = ""; };
$("#chat-cancel").onclick = () => activeRequest && api("/v1/chat/cancel", { request_id: activeRequest });
$("#chat-form").onsubmit = async ev => {
  ev.preventDefault();
  const text = $("#chat-input").value.trim();
  if (!text) return;
  $("#chat-input").value = "";
  addMsg("you", text, "user");
  const out = addMsg("model", "");
  try {
    if ($("#chat-session").checked && !session) session = (await api("/v1/chat/sessions", {})).session_id;
    activeRequest = "web-" + Math.random().toString(16).slice(2);
    const depth = $("#chat-depth").value;
    const body = { messages: [{ role: "user", content: text }], stream: true, request_id: activeRequest, max_tokens: +$("#chat-max").value,
      temperature: +$("#chat-temp").value, top_k: +$("#chat-topk").value, decode_depth: depth === "" ? null : +depth,
      speculative: $("#chat-spec").checked, session_id: $("#chat-session").checked ? session : null };
    $("#chat-send").disabled = true; $("#chat-cancel").disabled = false;
    const r = await fetch("/v1/chat/completions", { method: "POST", headers: { "Content-Type": "application/json" }, body: JSON.stringify(body) });
    if (!r.ok) throw new Error((await r.json()).detail || r.statusText);
    const reader = r.body.getReader(), dec = new TextDecoder();
    let buf = "";
    for (;;) {
      const { done, value } = await reader.read();
      if (done) break;
      buf += dec.decode(value, { stream: true });
      let cut;
      while ((cut = buf.indexOf("\n\n")) >= 0) {
        const line = buf.slice(0, cut).trim(); buf = buf.slice(cut + 2);
        if (!line.startsWith("data:")) continue;
        const payload = line.slice(5).trim();
        if (payload === "[DONE]") continue;
        const j = JSON.parse(payload);
        if (j.error) throw new Error(j.error);
        const d = j.choices && j.choices[0].delta;
        if (d && d.content) { out.textContent += d.content; $("#chat-log").scrollTop = 1e9; }
        if (j.telemetry) $("#chat-tele").textContent = Object.entries(j.telemetry).map(([k, v]) => `${k} ${fmt(v)}`).join("   ");
      }
    }
  } catch (e) { out.parentNode.classList.add("err"); out.textContent += " [" + e.message + "]"; }
  finally { $("#chat-send").disabled = false; $("#chat-cancel").disabled = true; activeRequest = null; }
};

// ---------------------------------------------------------------- training
function trainConfig() {
  return { lr: +$("#tr-lr").value, batch_size: +$("#tr-bs").value, seq_len: +$("#tr-seq").value, depth_mode: $("#tr-mode").value, grad_accum_steps: +$("#tr-accum").value };
}
function showTrain(s) {
  const t = s.error ? `error: ${s.error}` : `${s.running ? "running" : "idle"}   step ${s.step}   loss ${s.loss == null ? "-" : fmt(s.loss, 4)}   ${fmt(s.tok_s || 0)} tok/s`;
  say($("#tr-status"), t, !!s.error);
}
const trainCall = (path, body) => async () => { try { showTrain(await api(path, body ? body() : {})); } catch (e) { say($("#tr-status"), e.message, true); } };
$("#tr-start").onclick = trainCall("/v1/training/start", () => ({ config: trainConfig(), max_steps: +$("#tr-max").value || null }));
$("#tr-pause").onclick = trainCall("/v1/training/pause");
$("#tr-step").onclick = async () => { try { const s = await api("/v1/training/step", { config: trainConfig() }); lossSeries.push([s.step, s.loss]); drawLoss(); showTrain(s); } catch (e) { say($("#tr-status"), e.message, true); } };
$("#tr-save").onclick = async () => { try { const r = await api("/v1/checkpoints/save", { name: "studio_" + Date.now() }); say($("#tr-status"), "saved " + r.path); refreshCheckpoints(); } catch (e) { say($("#tr-status"), e.message, true); } };
function drawLoss() {
  const c = $("#tr-chart"), g = c.getContext("2d"), W = c.width, H = c.height;
  g.clearRect(0, 0, W, H);
  if (lossSeries.length < 2) return;
  const ys = lossSeries.map(p => p[1]).filter(Number.isFinite), lo = Math.min(...ys), hi = Math.max(...ys), span = hi - lo || 1;
  g.strokeStyle = "#2a323c"; g.fillStyle = "#8996a5"; g.font = "11px monospace";
  for (let k = 0; k <= 4; k++) { const y = 10 + (H - 30) * k / 4; g.beginPath(); g.moveTo(40, y); g.lineTo(W - 6, y); g.stroke(); g.fillText(fmt(hi - span * k / 4, 3), 2, y + 4); }
  g.strokeStyle = "#5fb3ff"; g.lineWidth = 1.5; g.beginPath();
  lossSeries.forEach((p, i) => { const x = 40 + (W - 46) * i / (lossSeries.length - 1), y = 10 + (H - 30) * (hi - p[1]) / span; i ? g.lineTo(x, y) : g.moveTo(x, y); });
  g.stroke();
  g.fillText("step " + lossSeries[0][0], 40, H - 4); g.fillText("step " + lossSeries[lossSeries.length - 1][0], W - 90, H - 4);
}
async function refreshCheckpoints() {
  try {
    const r = await api("/v1/checkpoints");
    const tb = $("#ck-table tbody"); tb.innerHTML = "";
    for (const c of r.checkpoints) {
      tb.append(el("tr", {}, el("td", {}, c.name || c.path), el("td", {}, String(c.step == null ? "" : c.step)), el("td", {}, c.size_bytes ? fmt(c.size_bytes / 1e6) + " MB" : ""),
        el("td", {}, el("button", { onclick: async () => { try { showActive(await api("/v1/checkpoints/load", { path: c.path })); } catch (e) { say($("#tr-status"), e.message, true); } } }, "Load"))));
    }
  } catch (e) { /* no directory yet */ }
}

// ---------------------------------------------------------------- fine-tuning
$("#ft-start").onclick = async () => {
  try {
    const records = $("#ft-records").value.split("\n").map(s => s.trim()).filter(Boolean).map(s => { try { return JSON.parse(s); } catch (e) { return s; } });
    const r = await api("/v1/finetune/start", { records, rank: +$("#ft-rank").value, alpha: +$("#ft-alpha").value, epochs: +$("#ft-epochs").value, lr: +$("#ft-lr").value,
      use_qlora: $("#ft-qlora").checked, output_dir: $("#ft-out").value });
    say($("#ft-status"), r.running ? "started" : JSON.stringify(r));
  } catch (e) { say($("#ft-status"), e.message, true); }
};
$("#ft-cancel").onclick = () => api("/v1/finetune/cancel", {}).then(() => say($("#ft-status"), "cancelling"));
$("#ft-merge").onclick = () => api("/v1/finetune/merge", {}).then(() => say($("#ft-status"), "merged"), e => say($("#ft-status"), e.message, true));
async function refreshAdapters() {
  const box = $("#ft-adapters"); box.innerHTML = "";
  try {
    const r = await api("/v1/finetune/adapters");
    if (!r.adapters.length) box.textContent = "none found under adapters/, checkpoints/, outputs/";
    for (const a of r.adapters) box.append(el("div", { class: "row" }, `${a.name}  r=${a.rank}`,
      el("button", { onclick: () => api("/v1/finetune/adapter", { action: "attach", path: a.path }).then(x => say($("#ft-status"), "attached " + x.active_adapter.name), e => say($("#ft-status"), e.message, true)) }, "Attach")));
    box.append(el("button", { onclick: () => api("/v1/finetune/adapter", { action: "detach" }).then(() => say($("#ft-status"), "detached")) }, "Detach"));
  } catch (e) { box.textContent = e.message; }
}

// ---------------------------------------------------------------- system
async function refreshSystem() {
  const put = (id, p) => api(p).then(d => $(id).textContent = JSON.stringify(d, null, 1), e => $(id).textContent = e.message);
  put("#sys-diag", "/v1/system/diagnostics"); put("#sys-vram", "/v1/vram/stats"); put("#sys-kernels", "/v1/engine/kernels");
}
$("#sys-purge").onclick = () => api("/v1/vram/purge", {}).then(refreshSystem);
$("#sys-turbo").onchange = e => api("/v1/engine/turbo_mode", { enabled: e.target.checked });

// ---------------------------------------------------------------- graph canvas
const graph = { nodes: [], edges: [] };
let catalog = null, selected = null, armed = null, seq = 1;
async function loadCatalog() {
  if (catalog) return;
  catalog = {};
  const r = await api("/v1/nodes/catalog");
  for (const n of r.studio_nodes) catalog[n.name] = n;
  renderPalette();
}
function renderPalette() {
  const f = $("#palette-filter").value.toLowerCase(), box = $("#palette-list"); box.innerHTML = "";
  const cats = {};
  for (const n of Object.values(catalog)) if (!f || n.name.toLowerCase().includes(f)) (cats[n.category] = cats[n.category] || []).push(n);
  for (const [c, list] of Object.entries(cats)) {
    box.append(el("div", { class: "cat" }, c));
    for (const n of list) box.append(el("button", { title: n.description, onclick: () => addNode(n.name) }, n.name));
  }
}
$("#palette-filter").oninput = renderPalette;
function addNode(kind, at, params, id) {
  const spec = catalog[kind];
  const n = { id: id || `${kind.toLowerCase()}_${seq++}`, type: spec ? spec.category : kind, title: kind, params: Object.assign({}, params || {}),
    x: at ? at[0] : 40 + (graph.nodes.length % 5) * 215, y: at ? at[1] : 30 + Math.floor(graph.nodes.length / 5) * 170 };
  graph.nodes.push(n); renderGraph(); select(n.id);
  return n;
}
function portsOf(n) {
  const s = catalog[n.title] || catalog[n.type];
  if (n.subgraph) return { ins: (n.subgraph.inputs || []).map(p => p.name), outs: (n.subgraph.outputs || []).map(p => p.name) };
  return s ? { ins: s.inputs, outs: s.outputs } : { ins: [], outs: [] };
}
function renderGraph() {
  const cv = $("#canvas"); cv.innerHTML = "";
  for (const n of graph.nodes) {
    const p = portsOf(n);
    const box = el("div", { class: "node" + (selected === n.id ? " sel" : "") + (n.status ? " " + n.status : ""), id: "node-" + n.id, style: `left:${n.x}px;top:${n.y}px` },
      el("div", { class: "title", onmousedown: e => startDrag(e, n) }, el("span", {}, `${n.title}`), el("span", { class: "x", onclick: e => { e.stopPropagation(); removeNode(n.id); } }, "×")),
      el("div", { class: "ports" },
        el("div", {}, ...p.ins.map(name => el("div", { class: "port in", "data-node": n.id, "data-port": name, onclick: e => clickPort(e, n.id, name, false) }, name))),
        el("div", {}, ...p.outs.map(name => el("div", { class: "port out" + (armed && armed.node === n.id && armed.port === name ? " armed" : ""), "data-node": n.id, "data-port": name, onclick: e => clickPort(e, n.id, name, true) }, name)))));
    box.addEventListener("mousedown", () => select(n.id));
    cv.append(box);
  }
  drawWires();
}
function removeNode(id) {
  graph.nodes = graph.nodes.filter(n => n.id !== id);
  graph.edges = graph.edges.filter(e => e.source !== id && e.target !== id);
  if (selected === id) { selected = null; $("#insp-body").textContent = "Select a node."; }
  renderGraph();
}
function clickPort(ev, node, port, isOut) {
  ev.stopPropagation();
  if (isOut) { armed = { node, port }; renderGraph(); return; }
  if (!armed) { graph.edges = graph.edges.filter(e => !(e.target === node && e.target_port === port)); renderGraph(); return; }  // click a bare input: disconnect it
  graph.edges = graph.edges.filter(e => !(e.target === node && e.target_port === port));  // one driver per input
  if (armed.node !== node) graph.edges.push({ source: armed.node, source_port: armed.port, target: node, target_port: port });
  armed = null; renderGraph();
}
function startDrag(ev, n) {
  const x0 = ev.clientX - n.x, y0 = ev.clientY - n.y;
  const move = e => { n.x = Math.max(0, e.clientX - x0); n.y = Math.max(0, e.clientY - y0); const d = $("#node-" + CSS.escape(n.id)); d.style.left = n.x + "px"; d.style.top = n.y + "px"; drawWires(); };
  const up = () => { document.removeEventListener("mousemove", move); document.removeEventListener("mouseup", up); };
  document.addEventListener("mousemove", move); document.addEventListener("mouseup", up);
}
function anchor(node, port, out) {
  const p = $(`.port.${out ? "out" : "in"}[data-node="${CSS.escape(node)}"][data-port="${CSS.escape(port)}"]`), w = $("#canvas-wrap");
  if (!p) { const d = $("#node-" + CSS.escape(node)); if (!d) return null; const r = d.getBoundingClientRect(), o = w.getBoundingClientRect(); return [r.left - o.left + w.scrollLeft + (out ? r.width : 0), r.top - o.top + w.scrollTop + 14]; }
  const r = p.getBoundingClientRect(), o = w.getBoundingClientRect();
  return [r.left - o.left + w.scrollLeft + (out ? r.width : 0), r.top - o.top + w.scrollTop + r.height / 2];
}
function drawWires() {
  const svg = $("#wires"); svg.innerHTML = "";
  for (const e of graph.edges) {
    const a = anchor(e.source, e.source_port || "", true), b = anchor(e.target, e.target_port || "", false);
    if (!a || !b) continue;
    const dx = Math.max(40, Math.abs(b[0] - a[0]) / 2);
    const path = document.createElementNS("http://www.w3.org/2000/svg", "path");
    path.setAttribute("d", `M${a[0]},${a[1]} C${a[0] + dx},${a[1]} ${b[0] - dx},${b[1]} ${b[0]},${b[1]}`);
    if (!e.source_port) path.setAttribute("class", "untyped");
    svg.append(path);
  }
}
function select(id) {
  selected = id;
  $$(".node").forEach(d => d.classList.toggle("sel", d.id === "node-" + id));
  const n = graph.nodes.find(x => x.id === id), box = $("#insp-body"); box.innerHTML = "";
  if (!n) return;
  const spec = catalog[n.title] || { parameters: {}, description: "" };
  box.append(el("div", {}, el("b", {}, n.title), " ", el("span", { class: "pill" }, n.id)), el("div", { class: "tele" }, spec.description || ""));
  const keys = Array.from(new Set([...Object.keys(spec.parameters || {}), ...Object.keys(n.params)]));
  for (const k of keys) {
    const cur = k in n.params ? n.params[k] : spec.parameters[k];
    const inp = el("input", { value: typeof cur === "string" ? cur : JSON.stringify(cur) });
    inp.onchange = () => { let v = inp.value; try { v = JSON.parse(v); } catch (e) { /* keep the text */ } n.params[k] = v; };
    box.append(el("label", {}, k), inp);
  }
  const nk = el("input", { placeholder: "new parameter name" });
  nk.onchange = () => { if (nk.value) { n.params[nk.value] = ""; select(id); } };
  box.append(el("label", {}, "add parameter"), nk);
  if (n.result) box.append(el("label", {}, "last result"), el("pre", { class: "small" }, JSON.stringify(n.result, null, 1)));
}
function exportGraph() {
  return { nodes: graph.nodes.map(n => { const o = { id: n.id, type: n.type, title: n.title, params: n.params, position: { x: n.x, y: n.y } }; if (n.subgraph) o.subgraph = n.subgraph; return o; }),
    edges: graph.edges.map(e => e.source_port ? e : { source: e.source, target: e.target }) };
}
function importGraph(g) {
  graph.nodes = (g.nodes || []).map((n, i) => ({ id: n.id, type: n.type, title: n.title || n.name || n.type, params: Object.assign({}, n.params || {}), subgraph: n.subgraph,
    x: (n.position && n.position.x) || n.x || 40 + (i % 5) * 215, y: (n.position && n.position.y) || n.y || 30 + Math.floor(i / 5) * 170 }));
  graph.edges = (g.edges || []).map(e => ({ source: e.source, target: e.target, source_port: e.source_port, target_port: e.target_port }));
  selected = null; renderGraph();
}
function onDagEvent(ev) {
  const n = graph.nodes.find(x => x.id === ev.node_id);
  if (!n) return;
  n.status = ev.event === "node_started" ? "running" : ev.event === "node_failed" ? "failed" : "completed";
  const d = $("#node-" + CSS.escape(n.id));
  if (d) d.className = "node " + n.status + (selected === n.id ? " sel" : "");
}
$("#g-run").onclick = async () => {
  graph.nodes.forEach(n => { n.status = ""; n.result = null; }); renderGraph();
  say($("#g-status"), "running…");
  try {
    const r = await api("/v1/dag/execute", exportGraph());
    for (const [id, res] of Object.entries(r.results || {})) { const n = graph.nodes.find(x => x.id === id); if (n) { n.status = res.status; n.result = res.output || { error: res.error }; } }
    renderGraph(); if (selected) select(selected);
    say($("#g-status"), r.status + (r.error ? ": " + r.error : ""), r.status === "failed");
    $("#g-output").textContent = JSON.stringify(r.results, null, 1);
  } catch (e) { say($("#g-status"), e.message, true); }
};
$("#g-compile").onclick = async () => { try { const r = await api("/v1/dag/compile_to_training", exportGraph()); say($("#g-status"), "compiled: " + r.sections.join(", ")); $("#g-output").textContent = JSON.stringify(r.applied, null, 1); refreshModels(); } catch (e) { say($("#g-status"), e.message, true); } };
$("#g-clear").onclick = () => { graph.nodes = []; graph.edges = []; selected = null; renderGraph(); };
$("#g-save").onclick = () => { const a = el("a", { href: URL.createObjectURL(new Blob([JSON.stringify(exportGraph(), null, 1)], { type: "application/json" })), download: "graph.json" }); a.click(); };
$("#g-open").onchange = async e => { const f = e.target.files[0]; if (f) { await loadCatalog(); importGraph(JSON.parse(await f.text())); } };
$("#g-demo").onclick = async () => {
  await loadCatalog();
  importGraph({ nodes: [
    { id: "model", type: "Model", title: "TriuneTransformer", params: { hidden_dim: 128, num_layers: 4, num_heads: 2, num_experts: 4, vocab_size: 256, use_node_config: true }, position: { x: 300, y: 40 } },
    { id: "tok", type: "Data", title: "BPETokenizer", params: {}, position: { x: 40, y: 40 } },
    { id: "opt", type: "Optimizer", title: "CentroidSteerOptimizer", params: { lr: 0.001 }, position: { x: 560, y: 40 } },
    { id: "step", type: "Evaluation", title: "TrainingStep", params: {}, position: { x: 820, y: 120 } },
    { id: "eval", type: "Evaluation", title: "PerplexityEvaluator", params: {}, position: { x: 1080, y: 120 } },
    { id: "text", type: "Runtime", title: "PythonSandbox", params: { code: "result = 'the quick brown fox jumps over the lazy dog ' * 4" }, position: { x: 40, y: 260 } } ],
  edges: [ { source: "text", source_port: "result", target: "tok", target_port: "text" }, { source: "tok", source_port: "tokens", target: "model", target_port: "input_ids" },
    { source: "model", source_port: "model_handle", target: "opt", target_port: "model_handle" }, { source: "model", source_port: "model_handle", target: "step", target_port: "model_handle" },
    { source: "opt", source_port: "optimizer_handle", target: "step", target_port: "optimizer_handle" }, { source: "tok", source_port: "tokens", target: "step", target_port: "tokens" },
    { source: "step", source_port: "model_handle", target: "eval", target_port: "model_handle" }, { source: "tok", source_port: "tokens", target: "eval", target_port: "tokens" } ] });
};
$("#canvas").addEventListener("click", () => { if (armed) { armed = null; renderGraph(); } });

refreshModels(); connectTelemetry(); api("/v1/training/status").then(showTrain, () => {});
