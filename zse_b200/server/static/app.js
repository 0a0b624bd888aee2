// Dashboard for the OpenAI-compatible server: streaming chat with stored sessions, LoRA adapters, retrieval
// documents, engine statistics and API keys.  Plain DOM code, no dependencies.
const $ = (id) => document.getElementById(id);
const auth = () => ($("key").value ? { Authorization: "Bearer " + $("key").value } : {});
const jsonHeaders = () => ({ "Content-Type": "application/json", ...auth() });
let history = [];
let session = null;           // id of the stored session the chat belongs to (null until the first message)
let aborter = null;

async function api(path, opts = {}) {
  const r = await fetch(path, { ...opts, headers: { ...(opts.body ? jsonHeaders() : auth()), ...(opts.headers || {}) } });
  const text = await r.text();
  let body = null;
  try { body = text ? JSON.parse(text) : null; } catch (e) { body = { error: text }; }
  return { ok: r.ok, status: r.status, body };
}

function el(tag, text, cls) {
  const e = document.createElement(tag);
  if (text !== undefined) e.textContent = text;
  if (cls) e.className = cls;
  return e;
}

function bubble(role, text) {
  const d = el("div", text, "msg " + role);
  $("log").appendChild(d);
  $("log").scrollTop = $("log").scrollHeight;
  return d;
}

// ---- status, models, statistics ------------------------------------------------------------------------------
async function refresh() {
  try {
    const h = await api("/health");
    $("status").textContent = h.ok ? `${h.body.model} (${h.body.engine})` : "offline";
    const keep = $("model").value;
    const m = await api("/v1/models");
    $("model").innerHTML = "";
    for (const x of (m.body && m.body.data) || []) $("model").appendChild(el("option", x.id));
    if (keep) $("model").value = keep;
    const s = await api("/v1/admin/stats");
    if (s.ok) $("stats").textContent = summary(s.body);
  } catch (e) { $("status").textContent = "offline"; }
}

function summary(s) {
  const e = s.engine || {}, kv = s.kv_cache || {}, sch = s.scheduler || {};
  const lines = [
    `requests ${e.total_requests ?? 0}, tokens out ${e.total_tokens_generated ?? 0}`,
    `running ${sch.active ?? sch.running ?? 0}, waiting ${sch.waiting ?? sch.queue_size ?? 0}`,
    `TTFT avg ${(e.avg_ttft_ms ?? 0).toFixed?.(1) ?? e.avg_ttft_ms} ms, TPOT avg ${(e.avg_tpot_ms ?? 0).toFixed?.(2) ?? e.avg_tpot_ms} ms`,
    `KV blocks ${kv.used_blocks ?? "?"}/${kv.total_blocks ?? "?"}, prefix hit rate ${kv.dedup_hit_rate ?? 0}`,
    `adapters ${(s.lora || {}).num_adapters ?? 0}, keys ${s.num_keys ?? 0}`,
  ];
  if (s.speculative) lines.push(`speculative acceptance ${JSON.stringify(s.speculative)}`);
  return lines.join("\n") + "\n\n" + JSON.stringify(s.usage || {}, null, 1);
}

// ---- sessions ------------------------------------------------------------------------------------------------
async function loadSessions() {
  const r = await api("/v1/dashboard/sessions");
  $("sessions").innerHTML = "";
  if (!r.ok) { $("sessions").appendChild(el("li", "enter a key to keep sessions", "hint")); return; }
  for (const s of r.body.sessions) {
    const li = el("li", "", s.session_id === session ? "active" : "");
    const open = el("a", `${new Date(s.updated_at * 1000).toLocaleString()} · ${s.messages} msgs`);
    open.href = "#";
    open.onclick = (ev) => { ev.preventDefault(); openSession(s.session_id); };
    const del = el("button", "×", "del");
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

function newChat() {
  session = null;
  history = [];
  $("log").innerHTML = "";
}

async function remember(role, content) {
  if (!$("key").value) return;
  if (!session) {
    const r = await api("/v1/dashboard/session", { method: "POST", body: "{}" });
    if (!r.ok) return;
    session = r.body.session_id;
  }
  const model = $("model").value || "";
  const [base, adapter] = model.split(":");
  await api(`/v1/dashboard/session/${session}/message`, { method: "POST",
    body: JSON.stringify({ role, content, model: base, lora_id: adapter || null }) });
}

// ---- chat ----------------------------------------------------------------------------------------------------
async function send() {
  const text = $("msg").value.trim();
  if (!text || aborter) return;
  $("msg").value = "";
  history.push({ role: "user", content: text });
  bubble("user", text);
  remember("user", text);
  const out = bubble("assistant", "");
  const messages = $("system").value ? [{ role: "system", content: $("system").value }, ...history] : history;
  aborter = new AbortController();
  $("stop").disabled = false;
  const t0 = performance.now();
  let first = 0, pieces = 0, full = "";
  try {
    const resp = await fetch("/v1/chat/completions", { method: "POST", headers: jsonHeaders(), signal: aborter.signal,
      body: JSON.stringify({ model: $("model").value, messages, stream: true, rag: $("rag").checked,
        max_tokens: +$("max").value, temperature: +$("temp").value, top_p: +$("topp").value }) });
    if (!resp.ok) { out.textContent = "error: " + (await resp.text()); out.classList.add("error"); return; }
    const reader = resp.body.getReader();
    const dec = new TextDecoder();
    let buf = "";
    for (;;) {
      const { done, value } = await reader.read();
      if (done) break;
      buf += dec.decode(value, { stream: true });
      let i;
      while ((i = buf.indexOf("\n\n")) >= 0) {
        const line = buf.slice(0, i); buf = buf.slice(i + 2);
        if (!line.startsWith("data: ") || line === "data: [DONE]") continue;
        const delta = JSON.parse(line.slice(6)).choices[0].delta || {};
        if (delta.content) {
          if (!first) first = performance.now();
          pieces += 1;
          full += delta.content;
          out.textContent = full;
          $("log").scrollTop = $("log").scrollHeight;
        }
      }
    }
  } catch (e) {
    if (e.name !== "AbortError") { out.textContent = full + "\n[" + e + "]"; out.classList.add("error"); }
  } finally {
    aborter = null;
    $("stop").disabled = true;
  }
  if (full) {
    history.push({ role: "assistant", content: full });
    await remember("assistant", full);
    const dt = (performance.now() - (first || t0)) / 1000;
    $("speed").textContent = `first token ${((first || t0) - t0).toFixed(0)} ms, ${(pieces / Math.max(dt, 1e-3)).toFixed(1)} pieces/s`;
  }
  loadSessions();
  refresh();
}

// ---- adapters ------------------------------------------------------------------------------------------------
async function loadAdapters() {
  const r = await api("/v1/lora/list");
  $("adapters").innerHTML = "";
  for (const a of (r.ok && r.body.adapters) || []) {
    const li = el("li", `${a.adapter_id} · rank ${a.rank} · ${(a.bytes / 1048576).toFixed(1)} MiB `);
    const rm = el("button", "unload", "del");
    rm.onclick = async () => { await api("/v1/lora/unload", { method: "POST", body: JSON.stringify({ adapter_id: a.adapter_id }) });
      loadAdapters(); refresh(); };
    li.appendChild(rm);
    $("adapters").appendChild(li);
  }
}

// ---- documents -----------------------------------------------------------------------------------------------
async function loadDocs() {
  const r = await api("/v1/rag/documents");
  $("docs").innerHTML = "";
  for (const d of (r.ok && r.body.documents) || []) {
    const li = el("li", `${d.name} · ${d.chunk_count} chunks · ${d.token_savings_pct}% fewer tokens `);
    const rm = el("button", "×", "del");
    rm.onclick = async () => { await api("/v1/rag/document/" + d.id, { method: "DELETE" }); loadDocs(); };
    li.appendChild(rm);
    $("docs").appendChild(li);
  }
}

function toBase64(buf) {
  let s = "";
  const b = new Uint8Array(buf);
  for (let i = 0; i < b.length; i += 0x8000) s += String.fromCharCode.apply(null, b.subarray(i, i + 0x8000));
  return btoa(s);
}

// ---- API keys ------------------------------------------------------------------------------------------------
async function loadKeys() {
  const r = await api("/v1/admin/keys/list");
  $("keys").innerHTML = "";
  for (const k of (r.ok && r.body.keys) || []) {
    const li = el("li", `${k.name || "(unnamed)"} · ${k.key_prefix || k.prefix || ""}… · ${k.rate_limit_rpm}/min ${k.is_active === false || k.active === false ? "· revoked" : ""} `);
    const rm = el("button", "revoke", "del");
    rm.onclick = async () => { await api("/v1/admin/keys/revoke", { method: "POST", body: JSON.stringify({ id: k.id }) }); loadKeys(); };
    li.appendChild(rm);
    $("keys").appendChild(li);
  }
}

// ---- wiring --------------------------------------------------------------------------------------------------
$("f").addEventListener("submit", (ev) => { ev.preventDefault(); send(); });
$("msg").addEventListener("keydown", (ev) => { if (ev.key === "Enter" && !ev.shiftKey) { ev.preventDefault(); send(); } });
$("stop").addEventListener("click", () => aborter && aborter.abort());
$("new").addEventListener("click", () => { newChat(); loadSessions(); });
$("theme").addEventListener("click", () => document.body.classList.toggle("light"));
$("lora").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const r = await api("/v1/lora/load", { method: "POST",
    body: JSON.stringify({ adapter_id: $("lora_id").value, path: $("lora_path").value }) });
  if (!r.ok) alert((r.body && (r.body.error && (r.body.error.message || r.body.error))) || "load failed");
  loadAdapters(); refresh();
});
$("up").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const f = $("file").files[0];
  if (!f) return;
  const body = { filename: f.name, content: toBase64(await f.arrayBuffer()) };
  if ($("pdfpw").value) body.pdf_password = $("pdfpw").value;
  const r = await api("/v1/rag/upload", { method: "POST", body: JSON.stringify(body) });
  if (!r.ok) alert((r.body && (r.body.error && (r.body.error.message || r.body.error))) || "upload failed");
  loadDocs();
});
$("search").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const r = await api("/v1/rag/search", { method: "POST", body: JSON.stringify({ query: $("query").value, top_k: 5 }) });
  $("hits").textContent = r.ok ? (r.body.results || []).map((h) =>
    `${Number(h.score || 0).toFixed(4)}  ${h.doc_name || ""}\n${(h.content || "").slice(0, 240)}`).join("\n\n")
    : "search failed";
});
$("mk").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const r = await api("/v1/admin/keys/create", { method: "POST",
    body: JSON.stringify({ name: $("kname").value, rate_limit_rpm: +($("krpm").value || 60) }) });
  $("newkey").textContent = r.ok ? "new key (shown once): " + r.body.key : "admin key required";
  loadKeys();
});
function everything() { refresh(); loadSessions(); loadAdapters(); loadDocs(); loadKeys(); }
$("key").addEventListener("change", everything);
everything();
setInterval(refresh, 15000);
