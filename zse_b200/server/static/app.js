// Minimal chat client for the OpenAI-compatible endpoint with SSE streaming.
const $ = (id) => document.getElementById(id);
const history = [];
const auth = () => ($("key").value ? { Authorization: "Bearer " + $("key").value } : {});

async function refresh() {
  try {
    const h = await (await fetch("/health")).json();
    $("status").textContent = `${h.model} (${h.engine})`;
    const m = await (await fetch("/v1/models", { headers: auth() })).json();
    $("model").innerHTML = (m.data || []).map((x) => `<option>${x.id}</option>`).join("");
    const s = await fetch("/v1/admin/stats", { headers: auth() });
    if (s.ok) $("stats").textContent = JSON.stringify(await s.json(), null, 1);
  } catch (e) { $("status").textContent = "offline"; }
}

function bubble(role, text) {
  const d = document.createElement("div");
  d.className = "msg " + role;
  d.textContent = text;
  $("log").appendChild(d);
  $("log").scrollTop = $("log").scrollHeight;
  return d;
}

$("f").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const text = $("msg").value.trim();
  if (!text) return;
  $("msg").value = "";
  history.push({ role: "user", content: text });
  bubble("user", text);
  const out = bubble("assistant", "");
  const resp = await fetch("/v1/chat/completions", {
    method: "POST", headers: { "Content-Type": "application/json", ...auth() },
    body: JSON.stringify({ model: $("model").value, messages: history, stream: true, rag: $("rag").checked,
      max_tokens: +$("max").value, temperature: +$("temp").value }) });
  if (!resp.ok) { out.textContent = "error: " + (await resp.text()); return; }
  const reader = resp.body.getReader();
  const dec = new TextDecoder();
  let buf = "", full = "";
  for (;;) {
    const { done, value } = await reader.read();
    if (done) break;
    buf += dec.decode(value, { stream: true });
    let i;
    while ((i = buf.indexOf("\n\n")) >= 0) {
      const line = buf.slice(0, i); buf = buf.slice(i + 2);
      if (!line.startsWith("data: ") || line === "data: [DONE]") continue;
      const delta = JSON.parse(line.slice(6)).choices[0].delta || {};
      if (delta.content) { full += delta.content; out.textContent = full; }
    }
  }
  history.push({ role: "assistant", content: full });
  refresh();
});
$("key").addEventListener("change", refresh);
refresh();
setInterval(refresh, 15000);
