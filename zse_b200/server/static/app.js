// Dashboard for the OpenAI-compatible server: streaming chat with stored sessions, raw completions, a live monitor
// (throughput, queue, latency, KV cache, speculative decoding), LoRA adapters, retrieval documents with search and a
// chunk viewer, API keys with per-key usage, and an inspector of the requests this page made (with the matching curl
// command).  Plain DOM code, no dependencies, no build step.
"use strict";
const $ = (id) => document.getElementById(id);
const auth = () => ($("key").value ? { Authorization: "Bearer " + $("key").value } : {});
const jsonHeaders = () => ({ "Content-Type": "application/json", ...auth() });
const store = {
  get(k, d) { try { const v = localStorage.getItem("zse." + k); return v === null ? d : JSON.parse(v); } catch (e) { return d; } },
  set(k, v) { try { localStorage.setItem("zse." + k, JSON.stringify(v)); } catch (e) { /* private mode */ } },
  del(k) { try { localStorage.removeItem("zse." + k); } catch (e) { /* private mode */ } },
};
let history = [];
let session = null;           // id of the stored session the chat belongs to (null until the first message)
let aborter = null;
let paused = false;
let timer = null;
const series = { tps: [], run: [], wait: [], ttft: [], tpot: [] };   // monitor history, newest last
let lastSample = null;        // {t, tokens} of the previous statistics sample
const calls = [];             // request inspector rows

// ---- small helpers -------------------------------------------------------------------------------------------
function el(tag, text, cls) {
  const e = document.createElement(tag);
  if (text !== undefined && text !== null) e.textContent = text;
  if (cls) e.className = cls;
  return e;
}
function td(row, text, cls) { const c = el("td", text, cls); row.appendChild(c); return c; }
function fmt(n, digits = 0) { return n === undefined || n === null || Number.isNaN(+n) ? "–" : (+n).toLocaleString(undefined, { maximumFractionDigits: digits }); }
function bytes(n) { return n >= 1 << 30 ? (n / (1 << 30)).toFixed(2) + " GiB" : n >= 1 << 20 ? (n / (1 << 20)).toFixed(1) + " MiB" : fmt(n / 1024, 1) + " KiB"; }
function when(ts) { return ts ? new Date(ts * 1000).toLocaleString() : "never"; }
function errText(r) { const b = r.body || {}; return (b.error && (b.error.message || b.error)) || b.message || ("HTTP " + r.status); }
function download(name, text, type) {
  const a = el("a");
  a.href = URL.createObjectURL(new Blob([text], { type }));
  a.download = name;
  a.click();
  setTimeout(() => URL.revokeObjectURL(a.href), 1000);
}

async function api(path, opts = {}, note) {
  const t0 = performance.now();
  const headers = { ...(opts.body ? jsonHeaders() : auth()), ...(opts.headers || {}) };
  let r, text = "";
  try {
    r = await fetch(path, { ...opts, headers });
    text = await r.text();
  } catch (e) {
    record(opts.method || "GET", path, opts.body, 0, String(e), performance.now() - t0);
    return { ok: false, status: 0, body: { error: String(e) } };
  }
  let body = null;
  try { body = text ? JSON.parse(text) : null; } catch (e) { body = { error: text }; }
  if (note !== false) record(opts.method || "GET", path, opts.body, r.status, text, performance.now() - t0);
  return { ok: r.ok, status: r.status, body };
}

// ---- markdown (a safe subset: code fences, inline code, bold, italics, links, lists, headings) ---------------
function escapeHtml(s) { return s.replace(/[&<>"]/g, (c) => ({ "&": "&amp;", "<": "&lt;", ">": "&gt;", '"': "&quot;" }[c])); }
function inlineMd(s) {
  return escapeHtml(s)
    .replace(/`([^`]+)`/g, "<code>$1</code>")
    .replace(/\*\*([^*]+)\*\*/g, "<b>$1</b>")
    .replace(/(^|[^*])\*([^*\n]+)\*/g, "$1<i>$2</i>")
    .replace(/\[([^\]]+)\]\((https?:\/\/[^\s)]+)\)/g, '<a href="$2" target="_blank" rel="noopener noreferrer">$1</a>');
}
function renderMd(text) {
  const out = [];
  const parts = text.split(/```/);
  parts.forEach((part, i) => {
    if (i % 2 === 1) {                                   // inside a fence: first line may name the language
      const nl = part.indexOf("\n");
      const lang = nl >= 0 ? part.slice(0, nl).trim() : "";
      const code = nl >= 0 ? part.slice(nl + 1) : part;
      out.push(`<div class="code"><span class="lang">${escapeHtml(lang)}</span><button class="copy" type="button">copy</button><pre>${escapeHtml(code)}</pre></div>`);
      return;
    }
    let list = null;
    for (const line of part.split("\n")) {
      const h = /^(#{1,4})\s+(.*)$/.exec(line);
      const li = /^\s*(?:[-*]|\d+\.)\s+(.*)$/.exec(line);
      if (li) {
        if (!list) { list = []; }
        list.push("<li>" + inlineMd(li[1]) + "</li>");
        continue;
      }
      if (list) { out.push("<ul>" + list.join("") + "</ul>"); list = null; }
      if (h) out.push(`<h${h[1].length + 2}>${inlineMd(h[2])}</h${h[1].length + 2}>`);
      else if (line.trim() === "") out.push("<br>");
      else out.push("<div>" + inlineMd(line) + "</div>");
    }
    if (list) out.push("<ul>" + list.join("") + "</ul>");
  });
  return out.join("");
}
function setBubble(d, text) {
  d.dataset.raw = text;
  if ($("md").checked && d.classList.contains("assistant")) d.innerHTML = renderMd(text);
  else d.textContent = text;
}
function bubble(role, text) {
  const d = el("div", "", "msg " + role);
  setBubble(d, text);
  $("log").appendChild(d);
  $("log").scrollTop = $("log").scrollHeight;
  return d;
}
document.addEventListener("click", (ev) => {
  if (ev.target.classList && ev.target.classList.contains("copy")) {
    const pre = ev.target.parentElement.querySelector("pre");
    navigator.clipboard && navigator.clipboard.writeText(pre.textContent);
    ev.target.textContent = "copied";
    setTimeout(() => { ev.target.textContent = "copy"; }, 1200);
  }
});

// ---- tabs ----------------------------------------------------------------------------------------------------
function show(tab) {
  for (const b of $("tabs").children) b.classList.toggle("on", b.dataset.tab === tab);
  for (const s of document.querySelectorAll("section.tab")) s.classList.toggle("on", s.id === "tab-" + tab);
  store.set("tab", tab);
  if (tab === "monitor") refresh();
  if (tab === "adapters") loadAdapters();
  if (tab === "documents") loadDocs();
  if (tab === "keys") { loadKeys(); }
  if (tab === "inspect") drawCalls();
}
$("tabs").addEventListener("click", (ev) => { if (ev.target.dataset.tab) show(ev.target.dataset.tab); });

// ---- status, models, statistics ------------------------------------------------------------------------------
function spark(canvas, rows, colors) {
  const c = canvas.getContext("2d");
  const w = canvas.width, h = canvas.height;
  c.clearRect(0, 0, w, h);
  const all = rows.flat();
  const top = Math.max(1e-9, ...all);
  rows.forEach((row, k) => {
    if (row.length < 2) return;
    c.beginPath();
    row.forEach((v, i) => {
      const x = (i / (row.length - 1)) * (w - 2) + 1, y = h - 2 - (v / top) * (h - 6);
      if (i === 0) c.moveTo(x, y); else c.lineTo(x, y);
    });
    c.strokeStyle = colors[k];
    c.lineWidth = 1.5;
    c.stroke();
  });
  c.fillStyle = getComputedStyle(document.body).color;
  c.font = "10px sans-serif";
  c.fillText(fmt(top, 1), 2, 10);
}
function push(name, v) { const s = series[name]; s.push(+v || 0); if (s.length > 120) s.shift(); }

async function refresh() {
  try {
    const h = await api("/health", {}, false);
    $("status").textContent = h.ok ? `${h.body.model} · ${h.body.engine}` : "offline";
    $("status").classList.toggle("bad", !h.ok);
    $("foot").textContent = h.ok ? `up ${fmt((h.body.uptime_s || 0) / 60, 1)} min` : "";
    const keepModel = $("model").value || store.get("model", "");
    const m = await api("/v1/models", {}, false);
    $("model").innerHTML = "";
    for (const x of (m.body && m.body.data) || []) $("model").appendChild(el("option", x.id));
    if (keepModel) $("model").value = keepModel;
    if (paused) return;
    const s = await api("/v1/admin/stats", {}, false);
    if (s.ok) monitor(s.body);
  } catch (e) { $("status").textContent = "offline"; $("status").classList.add("bad"); }
}

function monitor(s) {
  const e = s.engine || {}, kv = s.kv_cache || {}, sch = s.scheduler || {};
  const now = performance.now() / 1000, tokens = e.total_tokens_generated || 0;
  if (lastSample && now > lastSample.t) push("tps", Math.max(0, (tokens - lastSample.tokens) / (now - lastSample.t)));
  lastSample = { t: now, tokens };
  const running = sch.active ?? sch.running ?? sch.num_decoding ?? 0, waiting = sch.waiting ?? sch.queue_size ?? sch.num_waiting ?? 0;
  push("run", running); push("wait", waiting);
  push("ttft", e.p50_ttft_ms ?? e.avg_ttft_ms ?? 0); push("tpot", e.p50_tpot_ms ?? e.avg_tpot_ms ?? 0);
  $("m_tps").textContent = fmt(series.tps[series.tps.length - 1], 1);
  $("m_req").textContent = `${fmt(running)} / ${fmt(waiting)}`;
  $("m_req2").textContent = `running / waiting · ${fmt(e.total_requests)} served · ${fmt(tokens)} tokens out`;
  $("m_lat").textContent = `${fmt(e.p50_ttft_ms ?? e.avg_ttft_ms, 1)} / ${fmt(e.p50_tpot_ms ?? e.avg_tpot_ms, 2)}`;
  const used = kv.used_blocks ?? 0, total = kv.total_blocks ?? kv.num_total_blocks ?? 0;
  $("m_kv").textContent = total ? `${fmt(100 * used / total, 1)} %` : "–";
  $("b_kv").style.width = total ? `${Math.min(100, 100 * used / total)}%` : "0";
  $("m_kv2").textContent = `${fmt(used)} of ${fmt(total)} blocks · prefix hit rate ${fmt((kv.dedup_hit_rate ?? 0) * 100, 1)} % · ${fmt(kv.evictions ?? kv.num_evictions ?? 0)} evictions`;
  const sp = s.speculative;
  $("m_spec").textContent = sp ? `${fmt((sp.acceptance_rate ?? 0) * 100, 1)} %` : "–";
  $("m_spec2").textContent = sp ? `accepted ${fmt(sp.accepted ?? sp.total_accepted)} of ${fmt(sp.proposed ?? sp.total_proposed)} drafted tokens` : "off";
  const it = s.init_times || {};
  $("m_cold").textContent = it.total !== undefined ? `${fmt(it.total, 2)} s` : "–";
  $("m_cold2").textContent = it.total !== undefined ? `open ${fmt(it.open, 2)} · weights ${fmt(it.weights, 2)}${it.stream_gbs ? ` (${fmt(it.stream_gbs, 1)} GB/s)` : ""} · runtime ${fmt(it.runtime, 2)}` : "";
  spark($("c_tps"), [series.tps], ["#4aa3ff"]);
  spark($("c_run"), [series.run, series.wait], ["#4aa3ff", "#ffab40"]);
  spark($("c_lat"), [series.ttft, series.tpot], ["#4aa3ff", "#7bd88f"]);
  $("m_when").textContent = "updated " + new Date().toLocaleTimeString();
  $("stats").textContent = JSON.stringify(s, null, 1);
  $("lora_sum").textContent = `${(s.lora || {}).num_adapters ?? 0} loaded`;
}
function schedule() {
  if (timer) clearInterval(timer);
  timer = setInterval(refresh, 1000 * +$("every").value);
}
$("every").addEventListener("change", schedule);
$("pause").addEventListener("click", () => { paused = !paused; $("pause").textContent = paused ? "Resume" : "Pause"; });

// ---- sessions ------------------------------------------------------------------------------------------------
async function loadSessions() {
  const r = await api("/v1/dashboard/sessions", {}, false);
  $("sessions").innerHTML = "";
  if (!r.ok) { $("sessions").appendChild(el("li", "enter a key to keep sessions", "hint")); return; }
  const needle = $("sfilter").value.toLowerCase();
  for (const s of r.body.sessions) {
    const label = `${new Date(s.updated_at * 1000).toLocaleString()} · ${s.messages} msgs${s.title ? " · " + s.title : ""}`;
    if (needle && !label.toLowerCase().includes(needle)) continue;
    const li = el("li", "", s.session_id === session ? "active" : "");
    const open = el("a", label);
    open.href = "#";
    open.onclick = (ev) => { ev.preventDefault(); openSession(s.session_id); };
    const del = el("button", "×", "del");
    del.title = "delete this session";
    del.onclick = async () => { await api("/v1/dashboard/session/" + s.session_id, { method: "DELETE" });
      if (session === s.session_id) newChat(); loadSessions(); };
    li.append(open, del);
    $("sessions").appendChild(li);
  }
}
async function openSession(id) {
  const r = await api("/v1/dashboard/session/" + id);
  if (!r.ok) return;
  session = id;
  history = r.body.messages.map((m) => ({ role: m.role, content: m.content }));
  $("log").innerHTML = "";
  for (const m of history) bubble(m.role, m.content);
  loadSessions();
}
function newChat() { session = null; history = []; $("log").innerHTML = ""; $("speed").textContent = ""; }
async function remember(role, content) {
  if (!$("key").value) return;
  if (!session) {
    const r = await api("/v1/dashboard/session", { method: "POST", body: "{}" });
    if (!r.ok) return;
    session = r.body.session_id;
  }
  const [base, adapter] = ($("model").value || "").split(":");
  await api(`/v1/dashboard/session/${session}/message`, { method: "POST",
    body: JSON.stringify({ role, content, model: base, lora_id: adapter || null }) }, false);
}
$("sfilter").addEventListener("input", loadSessions);
$("export_json").addEventListener("click", () => download("chat.json", JSON.stringify({ model: $("model").value, messages: history }, null, 1), "application/json"));
$("export_md").addEventListener("click", () => download("chat.md", history.map((m) => `**${m.role}**\n\n${m.content}\n`).join("\n---\n\n"), "text/markdown"));
$("clear").addEventListener("click", () => { $("log").innerHTML = ""; });

// ---- chat ----------------------------------------------------------------------------------------------------
function samplingBody() {
  const b = { max_tokens: +$("max").value, temperature: +$("temp").value, top_p: +$("topp").value };
  if (+$("topk").value > 0) b.top_k = +$("topk").value;
  if (+$("rep").value !== 1) b.repetition_penalty = +$("rep").value;
  if ($("seed").value !== "") b.seed = +$("seed").value;
  return b;
}
async function streamInto(path, body, onPiece) {
  // returns {ok, status, text, first_ms, pieces, raw}
  const t0 = performance.now();
  const resp = await fetch(path, { method: "POST", headers: jsonHeaders(), signal: aborter.signal, body: JSON.stringify(body) });
  if (!resp.ok) { const text = await resp.text(); record("POST", path, JSON.stringify(body), resp.status, text, performance.now() - t0); return { ok: false, status: resp.status, text }; }
  let full = "", first = 0, pieces = 0, raw = "";
  if (!body.stream) {
    raw = await resp.text();
    const j = JSON.parse(raw);
    const c = j.choices[0];
    full = c.message ? c.message.content : c.text;
    onPiece(full);
    record("POST", path, JSON.stringify(body), resp.status, raw, performance.now() - t0, 0, 1);
    return { ok: true, text: full, first_ms: performance.now() - t0, pieces: 1, usage: j.usage };
  }
  const reader = resp.body.getReader();
  const dec = new TextDecoder();
  let buf = "";
  for (;;) {
    const { done, value } = await reader.read();
    if (done) break;
    const chunk = dec.decode(value, { stream: true });
    raw += chunk;
    buf += chunk;
    let i;
    while ((i = buf.indexOf("\n\n")) >= 0) {
      const line = buf.slice(0, i); buf = buf.slice(i + 2);
      if (!line.startsWith("data: ") || line === "data: [DONE]") continue;
      const ch = JSON.parse(line.slice(6)).choices[0];
      const piece = (ch.delta && ch.delta.content) || ch.text || "";
      if (piece) {
        if (!first) first = performance.now();
        pieces += 1;
        full += piece;
        onPiece(full);
      }
    }
  }
  record("POST", path, JSON.stringify(body), resp.status, raw.slice(-4000), performance.now() - t0, first ? first - t0 : 0, pieces);
  return { ok: true, text: full, first_ms: first ? first - t0 : 0, pieces, t0, first };
}
async function ask() {
  const out = bubble("assistant", "");
  const messages = $("system").value ? [{ role: "system", content: $("system").value }, ...history] : history;
  aborter = new AbortController();
  $("stop").disabled = false;
  let res = { ok: false, text: "" };
  try {
    res = await streamInto("/v1/chat/completions", { model: $("model").value, messages, stream: $("stream").checked,
      rag: $("rag").checked, ...samplingBody() }, (full) => { setBubble(out, full); $("log").scrollTop = $("log").scrollHeight; });
    if (!res.ok) { out.textContent = "error: " + res.text; out.classList.add("error"); }
  } catch (e) {
    if (e.name !== "AbortError") { out.textContent = (out.dataset.raw || "") + "\n[" + e + "]"; out.classList.add("error"); }
    res = { ok: true, text: out.dataset.raw || "", first_ms: 0, pieces: 0 };
  } finally {
    aborter = null;
    $("stop").disabled = true;
  }
  if (res.ok && res.text) {
    history.push({ role: "assistant", content: res.text });
    await remember("assistant", res.text);
    if (res.first) {
      const dt = (performance.now() - res.first) / 1000;
      $("speed").textContent = `first token ${res.first_ms.toFixed(0)} ms · ${(res.pieces / Math.max(dt, 1e-3)).toFixed(1)} pieces/s · ${res.pieces} pieces`;
    }
  }
  loadSessions();
}
async function send() {
  const text = $("msg").value.trim();
  if (!text || aborter) return;
  $("msg").value = "";
  history.push({ role: "user", content: text });
  bubble("user", text);
  remember("user", text);
  await ask();
}
async function regenerate() {
  if (aborter || !history.length) return;
  if (history[history.length - 1].role === "assistant") { history.pop(); const last = $("log").lastElementChild; if (last) last.remove(); }
  if (history.length) await ask();
}

// ---- raw completion ------------------------------------------------------------------------------------------
$("cf").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  if (aborter) return;
  aborter = new AbortController();
  $("cout").textContent = "";
  const body = { model: $("model").value, prompt: $("cprompt").value, stream: true, max_tokens: +$("cmax").value,
    temperature: +$("ctemp").value, echo: $("cecho").checked };
  if ($("cstop").value.trim()) body.stop = $("cstop").value.split(",").map((s) => s.trim()).filter(Boolean);
  const t0 = performance.now();
  try {
    const res = await streamInto("/v1/completions", body, (full) => { $("cout").textContent = full; });
    if (!res.ok) $("cout").textContent = "error: " + res.text;
    else $("cspeed").textContent = `${res.pieces} pieces in ${((performance.now() - t0) / 1000).toFixed(2)} s`;
  } catch (e) { if (e.name !== "AbortError") $("cout").textContent += "\n[" + e + "]"; }
  aborter = null;
});

// ---- adapters ------------------------------------------------------------------------------------------------
async function loadAdapters() {
  const r = await api("/v1/lora/list", {}, false);
  const body = $("adapters").tBodies[0];
  body.innerHTML = "";
  for (const a of (r.ok && r.body.adapters) || []) {
    const tr = el("tr");
    td(tr, a.adapter_id); td(tr, a.rank); td(tr, a.alpha); td(tr, (a.target_modules || []).join(", ")); td(tr, bytes(a.bytes || 0));
    const use = el("button", "use");
    use.title = "select model:adapter for the chat";
    use.onclick = () => { const base = ($("model").value || "").split(":")[0]; const id = `${base}:${a.adapter_id}`;
      if (![...$("model").options].some((o) => o.value === id)) $("model").appendChild(el("option", id)); $("model").value = id; store.set("model", id); };
    const rm = el("button", "unload", "del");
    rm.onclick = async () => { await api("/v1/lora/unload", { method: "POST", body: JSON.stringify({ adapter_id: a.adapter_id }) }); loadAdapters(); refresh(); };
    const c = td(tr, ""); c.append(use, rm);
    body.appendChild(tr);
  }
  if (!body.children.length) { const tr = el("tr"); const c = td(tr, r.ok ? "no adapter is loaded" : errText(r), "hint"); c.colSpan = 6; body.appendChild(tr); }
}
$("lora").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const r = await api("/v1/lora/load", { method: "POST", body: JSON.stringify({ adapter_id: $("lora_id").value, path: $("lora_path").value }) });
  if (!r.ok) alert(errText(r));
  loadAdapters(); refresh();
});

// ---- documents -----------------------------------------------------------------------------------------------
async function loadDocs() {
  const r = await api("/v1/rag/documents", {}, false);
  const body = $("docs").tBodies[0];
  body.innerHTML = "";
  for (const d of (r.ok && r.body.documents) || []) {
    const tr = el("tr");
    const name = td(tr, ""); const a = el("a", d.name); a.href = "#"; a.onclick = (ev) => { ev.preventDefault(); showDoc(d.id, d.name); }; name.appendChild(a);
    td(tr, d.doc_type || d.type || ""); td(tr, d.chunk_count); td(tr, `${d.token_savings_pct ?? 0} %`);
    const rm = el("button", "×", "del");
    rm.onclick = async () => { await api("/v1/rag/document/" + d.id, { method: "DELETE" }); loadDocs(); };
    td(tr, "").appendChild(rm);
    body.appendChild(tr);
  }
  const st = await api("/v1/rag/stats", {}, false);
  if (st.ok) $("rag_sum").textContent = `${st.body.documents ?? st.body.num_documents ?? 0} documents · ${st.body.chunks ?? st.body.num_chunks ?? 0} chunks`;
}
async function showDoc(id, name) {
  const r = await api("/v1/rag/document/" + id);
  $("docname").textContent = name;
  $("chunks").innerHTML = "";
  if (!r.ok) { $("chunks").textContent = errText(r); return; }
  const chunks = r.body.chunks || [];
  if (!chunks.length) { $("chunks").textContent = JSON.stringify(r.body, null, 1); return; }
  chunks.forEach((c, i) => {
    const d = el("div", "", "chunk");
    d.appendChild(el("span", `#${c.index ?? i}${c.page ? " · p." + c.page : ""} · ${c.token_count ?? "?"} tokens`, "hint"));
    d.appendChild(el("div", c.content || c.text || ""));
    $("chunks").appendChild(d);
  });
}
function toBase64(buf) {
  let s = "";
  const b = new Uint8Array(buf);
  for (let i = 0; i < b.length; i += 0x8000) s += String.fromCharCode.apply(null, b.subarray(i, i + 0x8000));
  return btoa(s);
}
async function uploadFiles(files) {
  let done = 0;
  for (const f of files) {
    $("upmsg").textContent = `uploading ${f.name}…`;
    const body = { filename: f.name, content: toBase64(await f.arrayBuffer()) };
    if ($("pdfpw").value) body.pdf_password = $("pdfpw").value;
    const r = await api("/v1/rag/upload", { method: "POST", body: JSON.stringify(body) });
    if (!r.ok) { $("upmsg").textContent = `${f.name}: ${errText(r)}`; continue; }
    done += 1;
  }
  $("upmsg").textContent = `${done} of ${files.length} uploaded`;
  loadDocs();
}
$("up").addEventListener("submit", (ev) => { ev.preventDefault(); if ($("file").files.length) uploadFiles([...$("file").files]); });
$("drop").addEventListener("dragover", (ev) => { ev.preventDefault(); $("drop").classList.add("over"); });
$("drop").addEventListener("dragleave", () => $("drop").classList.remove("over"));
$("drop").addEventListener("drop", (ev) => { ev.preventDefault(); $("drop").classList.remove("over"); uploadFiles([...ev.dataTransfer.files]); });
function highlight(text, query) {
  const words = query.toLowerCase().split(/\W+/).filter((w) => w.length > 2);
  let html = escapeHtml(text);
  for (const w of words) html = html.replace(new RegExp("(" + w.replace(/[.*+?^${}()|[\]\\]/g, "\\$&") + ")", "gi"), "<mark>$1</mark>");
  return html;
}
$("search").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const mode = $("smode").value, q = $("query").value;
  const body = { query: q, top_k: +$("stop_k").value };
  if (mode === "bm25") body.use_dense = false;
  if (mode === "dense") { body.use_dense = true; body.fusion = "weighted"; }
  const r = await api("/v1/rag/search", { method: "POST", body: JSON.stringify(body) });
  $("hits").innerHTML = "";
  if (!r.ok) { $("hits").textContent = errText(r); return; }
  for (const h of r.body.results || []) {
    const d = el("div", "", "hit");
    d.appendChild(el("span", `${Number(h.score || 0).toFixed(4)} · ${h.doc_name || ""}${h.page ? " · p." + h.page : ""}`, "hint"));
    const t = el("div"); t.innerHTML = highlight((h.content || "").slice(0, 600), q); d.appendChild(t);
    $("hits").appendChild(d);
  }
  if (!(r.body.results || []).length) $("hits").textContent = "nothing found";
});

// ---- API keys and usage --------------------------------------------------------------------------------------
async function loadKeys() {
  const r = await api("/v1/admin/keys/list", {}, false);
  const body = $("keys").tBodies[0], ubody = $("usage").tBodies[0];
  body.innerHTML = ""; ubody.innerHTML = "";
  if (!r.ok) { const tr = el("tr"); const c = td(tr, "an admin key lists the keys", "hint"); c.colSpan = 6; body.appendChild(tr); return; }
  const bars = [];
  for (const k of r.body.keys || []) {
    const tr = el("tr");
    td(tr, k.name || "(unnamed)"); td(tr, (k.prefix || k.key_prefix || "") + "…");
    const rpm = el("input"); rpm.type = "number"; rpm.value = k.rate_limit_rpm; rpm.min = 1; rpm.className = "narrow";
    rpm.onchange = async () => { const u = await api("/v1/admin/keys/update", { method: "POST", body: JSON.stringify({ id: k.id, rate_limit_rpm: +rpm.value }) }); if (!u.ok) alert(errText(u)); };
    td(tr, "").appendChild(rpm);
    td(tr, k.is_active === false ? "revoked" : "active", k.is_active === false ? "bad" : "");
    td(tr, `${fmt(k.total_requests)} requests · ${fmt(k.total_tokens)} tokens`);
    const rm = el("button", "revoke", "del");
    rm.disabled = k.is_active === false;
    rm.onclick = async () => { if (confirm(`revoke ${k.name || k.prefix}?`)) { await api("/v1/admin/keys/revoke", { method: "POST", body: JSON.stringify({ id: k.id }) }); loadKeys(); } };
    td(tr, "").appendChild(rm);
    body.appendChild(tr);
    const u = await api("/v1/admin/usage?key_id=" + k.id, {}, false);
    if (u.ok) {
      const ur = el("tr");
      td(ur, k.name || k.prefix); td(ur, fmt(u.body.total_requests)); td(ur, fmt(u.body.prompt_tokens)); td(ur, fmt(u.body.completion_tokens)); td(ur, `${fmt(u.body.avg_latency_ms, 1)} ms`);
      ubody.appendChild(ur);
      bars.push({ name: k.name || k.prefix, v: u.body.total_tokens || 0 });
    }
  }
  const c = $("c_usage").getContext("2d"), w = $("c_usage").width, h = $("c_usage").height;
  c.clearRect(0, 0, w, h);
  const top = Math.max(1, ...bars.map((b) => b.v));
  c.font = "10px sans-serif";
  bars.slice(0, 10).forEach((b, i) => {
    const bw = Math.max(1, (b.v / top) * (w - 120));
    c.fillStyle = "#4aa3ff"; c.fillRect(110, 4 + i * 11, bw, 8);
    c.fillStyle = getComputedStyle(document.body).color; c.fillText(String(b.name).slice(0, 18), 2, 11 + i * 11);
  });
}
$("mk").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const r = await api("/v1/admin/keys/create", { method: "POST", body: JSON.stringify({ name: $("kname").value,
    rate_limit_rpm: +($("krpm").value || 60), is_admin: $("kadmin").checked }) });
  $("newkey").textContent = r.ok ? "new key (shown once, copy it now):\n" + r.body.key : errText(r);
  loadKeys();
});

// ---- request inspector ---------------------------------------------------------------------------------------
function record(method, path, body, status, text, ms, first, pieces) {
  calls.unshift({ t: new Date(), method, path, body: body || "", status, text: String(text || "").slice(0, 20000), ms, first: first || 0, pieces: pieces || 0 });
  if (calls.length > 100) calls.pop();
  if (document.querySelector("#tab-inspect.on")) drawCalls();
}
function drawCalls() {
  const body = $("reqs").tBodies[0];
  body.innerHTML = "";
  calls.forEach((c) => {
    const tr = el("tr");
    td(tr, c.t.toLocaleTimeString()); td(tr, `${c.method} ${c.path}`); td(tr, c.status || "failed", c.status >= 400 || !c.status ? "bad" : "");
    td(tr, fmt(c.ms, 0)); td(tr, c.first ? fmt(c.first, 0) + " ms" : ""); td(tr, c.pieces || "");
    tr.onclick = () => {
      let pretty = c.body;
      try { pretty = JSON.stringify(JSON.parse(c.body), null, 1); } catch (e) { /* not JSON */ }
      $("req_body").textContent = pretty;
      let resp = c.text;
      try { resp = JSON.stringify(JSON.parse(c.text), null, 1); } catch (e) { /* a stream */ }
      $("resp_body").textContent = resp;
      const keyPart = $("key").value ? ` -H "Authorization: Bearer $ZSE_API_KEY"` : "";
      $("curl").textContent = `curl -sN ${location.origin}${c.path} -X ${c.method}${keyPart}` + (c.body ? ` -H "Content-Type: application/json" -d '${c.body.replace(/'/g, "'\\''")}'` : "");
    };
    body.appendChild(tr);
  });
}
$("wipe").addEventListener("click", () => { calls.length = 0; drawCalls(); });

// ---- wiring --------------------------------------------------------------------------------------------------
$("f").addEventListener("submit", (ev) => { ev.preventDefault(); send(); });
$("msg").addEventListener("keydown", (ev) => { if (ev.key === "Enter" && !ev.shiftKey) { ev.preventDefault(); send(); } });
$("stop").addEventListener("click", () => aborter && aborter.abort());
$("regen").addEventListener("click", regenerate);
$("new").addEventListener("click", () => { newChat(); loadSessions(); });
$("md").addEventListener("change", () => { for (const d of $("log").children) setBubble(d, d.dataset.raw || d.textContent); });
function setTheme(light) { document.body.classList.toggle("light", light); store.set("light", light); }
$("theme").addEventListener("click", () => setTheme(!document.body.classList.contains("light")));
$("model").addEventListener("change", () => store.set("model", $("model").value));
$("keep").addEventListener("change", () => { if ($("keep").checked) store.set("key", $("key").value); else store.del("key"); });
document.addEventListener("keydown", (ev) => {
  if (ev.key === "Escape" && aborter) aborter.abort();
  if (["INPUT", "TEXTAREA", "SELECT"].includes(document.activeElement.tagName)) return;
  if (ev.key === "n") { newChat(); loadSessions(); }
  if (ev.key === "t") setTheme(!document.body.classList.contains("light"));
  const tabs = [...$("tabs").children];
  if (/^[1-7]$/.test(ev.key) && tabs[+ev.key - 1]) show(tabs[+ev.key - 1].dataset.tab);
});
function everything() { refresh(); loadSessions(); loadAdapters(); loadDocs(); loadKeys(); }
$("key").addEventListener("change", () => { if ($("keep").checked) store.set("key", $("key").value); everything(); });
(function start() {
  setTheme(store.get("light", false));
  const k = store.get("key", "");
  if (k) { $("key").value = k; $("keep").checked = true; }
  for (const id of ["max", "temp", "topp", "topk", "rep", "system"]) {
    const v = store.get("p." + id, null);
    if (v !== null) $(id).value = v;
    $(id).addEventListener("change", () => store.set("p." + id, $(id).value));
  }
  show(store.get("tab", "chat"));
  everything();
  schedule();
})();
